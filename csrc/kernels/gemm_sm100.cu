// Plain bf16 GEMM entry point on the tcgen05 / TMEM / TMA pipeline of gemm_sm100.cuh.
// Replaces the cuBLAS calls of the reference (src/backend/gpu_native/math/gemm.cu:3-189) and the
// backward GEMM pair of src/ops/linear.cpp:30-68, with bias / GELU / residual / accumulate epilogues.
#include "gemm_sm100.cuh"

namespace lt {

template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  gemm_body<BLOCK_N, A_MAJOR, B_MAJOR>(&tmA, &tmB, p, NoGate(), NoDone());
}

template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BLOCK_N, A_MAJOR, B_MAJOR>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(tmA, tmB, p);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // namespace lt

extern "C" {

// C[M,N] = epilogue(alpha * op(A) * op(B)).  See gemm_sm100.cuh for the operand layouts.
// lda/ldb/ldc/ldr are pitches in elements. block_n: 0 = choose, else 128 or 256. max_ctas: 0 = one per SM.
// Returns 0, a cudaError_t, or 1000+/2000+ CUresult when a tensor map could not be encoded.
int lt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                 long long ldr, int act, int accumulate, float alpha, int block_n, int max_ctas, void* stream) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda * 2) % 16 != 0 || (ldb * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  if (block_n != 128 && block_n != 256) block_n = pick_block_n(M, N, sms);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.act = act; p.accumulate = accumulate; p.alpha = alpha;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  CUtensorMap tmA, tmB;
  int r = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_major, b_major, block_n);
  if (r) return r;
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > p.num_tiles) grid = p.num_tiles;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int key = (block_n == 256 ? 4 : 0) | (a_major ? 2 : 0) | (b_major ? 1 : 0);
  switch (key) {
    case 0: return launch_gemm<128, 0, 0>(tmA, tmB, p, grid, st);
    case 1: return launch_gemm<128, 0, 1>(tmA, tmB, p, grid, st);
    case 2: return launch_gemm<128, 1, 0>(tmA, tmB, p, grid, st);
    case 3: return launch_gemm<128, 1, 1>(tmA, tmB, p, grid, st);
    case 4: return launch_gemm<256, 0, 0>(tmA, tmB, p, grid, st);
    case 5: return launch_gemm<256, 0, 1>(tmA, tmB, p, grid, st);
    case 6: return launch_gemm<256, 1, 0>(tmA, tmB, p, grid, st);
    default: return launch_gemm<256, 1, 1>(tmA, tmB, p, grid, st);
  }
}

}  // extern "C"
