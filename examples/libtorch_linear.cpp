// The device library from C++ with libtorch as the tensor layer: a module whose forward pass is one call of the
// tcgen05 GEMM (bias and GELU in its epilogue), checked against libtorch's own matmul.  This is the C++ counterpart of
// `ops.functional.linear`: libtorch owns the memory and the stream, liblt_cuda.so does the math.
//
//   cmake -S . -B build/cmake -DLT_BUILD_LIBTORCH_EXAMPLE=ON -DCMAKE_PREFIX_PATH=$(python -c "import torch; print(torch.utils.cmake_prefix_path)")
//   cmake --build build/cmake -j --target lt_libtorch_linear && ./build/cmake/lt_libtorch_linear        # needs a B200
#include <c10/cuda/CUDAStream.h>
#include <torch/torch.h>

#include <cstdio>

#include "lt_cuda.h"

struct LtLinear : torch::nn::Module {
  torch::Tensor weight, bias;   // [out, in] and [out], bf16
  bool gelu;

  LtLinear(int64_t in, int64_t out, bool gelu_) : gelu(gelu_) {
    const auto opt = torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA);
    weight = register_parameter("weight", (torch::randn({out, in}, opt) * 0.02).detach());
    bias = register_parameter("bias", torch::zeros({out}, opt));
  }

  // x: [M, in] bf16, contiguous.  K-major operands on both sides (a_major = b_major = 0): y = act(x W^T + b).
  torch::Tensor forward(const torch::Tensor& x) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 2, "x: [M, K] bf16 on the device");
    const int M = int(x.size(0)), K = int(x.size(1)), N = int(weight.size(0));
    TORCH_CHECK(K == weight.size(1) && K % 8 == 0 && N % 8 == 0, "K and N must be multiples of 8 (16-byte rows for TMA)");
    auto y = torch::empty({M, N}, x.options());
    void* stream = c10::cuda::getCurrentCUDAStream().stream();
    const int rc = lt_gemm_bf16(x.data_ptr(), weight.data_ptr(), y.data_ptr(), M, N, K, /*lda*/ K, /*ldb*/ K, /*ldc*/ N,
                                /*a_major*/ 0, /*b_major*/ 0, /*out_fp32*/ 0, bias.data_ptr(), /*residual*/ nullptr, /*ldr*/ 0,
                                /*act*/ gelu ? 1 : 0, /*accumulate*/ 0, /*alpha*/ 1.0f, /*block_n*/ 0, /*max_ctas*/ 0, stream);
    TORCH_CHECK(rc == 0, "lt_gemm_bf16 returned ", rc);
    return y;
  }
};

int main() {
  if (!torch::cuda::is_available()) {
    std::printf("no CUDA device: nothing to run\n");
    return 0;
  }
  torch::manual_seed(0);
  LtLinear layer(4096, 11008, /*gelu*/ true);
  const auto x = torch::randn({2048, 4096}, torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA));
  const auto y = layer.forward(x);
  const auto ref = torch::gelu(torch::matmul(x.to(torch::kFloat), layer.weight.to(torch::kFloat).t()) + layer.bias.to(torch::kFloat), "tanh");
  torch::cuda::synchronize();
  const int status = lt_status_fetch();                       // non-zero: a bounded wait inside the kernel ran out
  const double err = (y.to(torch::kFloat) - ref).abs().max().item<double>();
  std::printf("max |lt - torch| = %.4g (bf16 output), device status %d\n", err, status);
  return (status == 0 && err < 0.05) ? 0 : 1;
}
