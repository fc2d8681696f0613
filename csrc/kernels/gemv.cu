// Weight-streaming GEMM for a handful of rows (decode with 1-8 sequences): y[M, N] = x[M, K] @ W[N, K]^T (+ residual).
//
// With so few rows the multiplication is bound by reading W once; 128-row tensor-core tiles waste the tile's rows and,
// for narrow outputs, leave most SMs without a tile.  Here a warp owns one output column (one row of W): its lanes walk
// the row in 16-byte steps, four loads in flight per lane, and keep one partial dot product per input row; a shuffle
// reduction finishes the column.  x (a few KB) is read through the read-only path and stays in L1.  The reference runs
// every Linear through cublasSgemm whatever the row count (src/ops/linear.cpp:176-192).
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kGemvMaxM = 8;
constexpr int kGemvWarps = 8;

template <int M>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w, long long ldw,
                 __nv_bfloat16* __restrict__ y, long long ldy, const __nv_bfloat16* __restrict__ residual, long long ldr,
                 int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int n = blockIdx.x * kGemvWarps + warp; n < N; n += gridDim.x * kGemvWarps) {
    const __nv_bfloat16* wr = w + (long long)n * ldw;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    // K is a multiple of 8; a lane takes 8 elements per step, the warp 256
    for (int k0 = lane * 8; k0 < K; k0 += 4 * 256) {
      uint4 wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 256;
        wv[u] = (k < K) ? ld_nc_v4(wr + k) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 256;
        if (k >= K) break;
        const float2 w0 = unpack_bf16x2(wv[u].x), w1 = unpack_bf16x2(wv[u].y), w2 = unpack_bf16x2(wv[u].z), w3 = unpack_bf16x2(wv[u].w);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (long long)m * ldx + k));
          const float2 x0 = unpack_bf16x2(xv.x), x1 = unpack_bf16x2(xv.y), x2 = unpack_bf16x2(xv.z), x3 = unpack_bf16x2(xv.w);
          acc[m] += w0.x * x0.x + w0.y * x0.y + w1.x * x1.x + w1.y * x1.y + w2.x * x2.x + w2.y * x2.y + w3.x * x3.x + w3.y * x3.y;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[m];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) {
        if (residual) v += __bfloat162float(residual[(long long)m * ldr + n]);
        y[(long long)m * ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

}  // namespace lt

extern "C" {

// y[M, N] = x[M, K] @ w[N, K]^T (+ residual[M, N]); 1 <= M <= 8, K a multiple of 8, rows 16-byte aligned.
int lt_gemv_bf16(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy, const void* residual,
                 long long ldr, int M, int N, int K, void* stream) {
  using namespace lt;
  if (M < 1 || M > kGemvMaxM || N <= 0 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  int blocks = (N + kGemvWarps - 1) / kGemvWarps;
  if (blocks > sms * 8) blocks = sms * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto R = static_cast<const __nv_bfloat16*>(residual);
#define LT_GEMV(MM) gemv_bf16_kernel<MM><<<blocks, kGemvWarps * 32, 0, st>>>(X, ldx, W, ldw, Y, ldy, R, ldr, N, K)
  switch (M) {
    case 1: LT_GEMV(1); break;
    case 2: LT_GEMV(2); break;
    case 3: LT_GEMV(3); break;
    case 4: LT_GEMV(4); break;
    case 5: LT_GEMV(5); break;
    case 6: LT_GEMV(6); break;
    case 7: LT_GEMV(7); break;
    default: LT_GEMV(8); break;
  }
#undef LT_GEMV
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
