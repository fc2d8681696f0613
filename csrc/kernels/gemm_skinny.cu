// Weight-streaming GEMM for 9 to 128 rows (decode with a batch of sequences): y[M, N] = x[M, K] @ W[N, K]^T (+ residual).
//
// With this few rows the multiplication is bound by reading W once (a 1.1B model's weights stream in 0.3 ms), but a
// 128-row tcgen05 tile wastes most of its rows and, worse, a 2048-column output gives a persistent tile kernel 8 or 16
// tiles for 148 SMs.  Here a CTA of eight warps owns 32 output columns and a slice of K; every warp walks its share of the
// slice in 32-element chunks with 8 to 16 sixteen-byte weight loads in flight per lane and feeds them to the warp-level
// tensor-core instruction (mma.sync m16n8k16: 16 rows of x by 8 columns of W; tcgen05's smallest tile is 64 rows and needs a
// TMEM / barrier set-up that costs more than these microsecond kernels run).  The K dimension inside a chunk is permuted
// the same way for both operands so that each lane's 16 contiguous bytes are exactly its fragments of two instructions.
// The eight warps' partial sums are folded through shared memory; when several CTAs share a column group (narrow
// outputs: more CTAs than column groups are needed to fill the GPU) each writes its partial to a workspace and the CTA
// that arrives last at the group's counter adds them in a fixed order, so the result does not depend on arrival order
// and nothing ever waits.  The reference runs every Linear through cublasSgemm whatever the row count
// (src/ops/linear.cpp:176-192).
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace lt {

constexpr int kSkWarps = 8;
constexpr int kSkCols = 32;   // output columns per CTA: four 8-column fragments per warp
constexpr size_t kSkWsBytes = 12u << 20;
constexpr int kSkCounters = 4096;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT = number of 16-row blocks of x (rows past M read as zero).  Grid: (column groups, K splits).
template <int MT>
__global__ void __launch_bounds__(kSkWarps * 32, 1)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w, long long ldw,
                   __nv_bfloat16* __restrict__ y, long long ldy, const __nv_bfloat16* __restrict__ residual, long long ldr,
                   int M, int N, int K, int chunks_per_cta, float* __restrict__ ws, unsigned* __restrict__ counters) {
  extern __shared__ float red[];   // [4 slots][MT * 16 registers][32 lanes]
  constexpr int R = MT * 16;
  constexpr int U = MT <= 2 ? 4 : 2;   // chunks whose weight loads are in flight together
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * kSkCols;
  const int nchunks = K >> 5;
  const int c_begin = blockIdx.y * chunks_per_cta;
  const int c_end = min(nchunks, c_begin + chunks_per_cta);

  float acc[MT][4][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int f = 0; f < 4; ++f)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[m][f][r] = 0.f;

  const __nv_bfloat16* wrow[4];
  bool wok[4];
#pragma unroll
  for (int f = 0; f < 4; ++f) {
    const int n = n0 + f * 8 + g;
    wok[f] = n < N;
    wrow[f] = w + (long long)(wok[f] ? n : 0) * ldw + q * 8;
  }
  const __nv_bfloat16* xbase = x + q * 8;

  for (int c = c_begin + warp; c < c_end; c += kSkWarps * U) {
    uint4 wv[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int cc = c + u * kSkWarps;
#pragma unroll
      for (int f = 0; f < 4; ++f)
        wv[u][f] = (cc < c_end && wok[f]) ? ld_nc_v4(wrow[f] + (long long)cc * 32) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int cc = c + u * kSkWarps;
      if (cc >= c_end) break;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const int r0 = m * 16 + g, r1 = r0 + 8;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const uint4 xlo = r0 < M ? __ldg(reinterpret_cast<const uint4*>(xbase + (long long)r0 * ldx + cc * 32)) : zero;
        const uint4 xhi = r1 < M ? __ldg(reinterpret_cast<const uint4*>(xbase + (long long)r1 * ldx + cc * 32)) : zero;
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          // physical k = q * 8 + j * 4 + {0, 1} plays logical k = q * 2 + {0, 1}, physical + 2 plays logical + 8, for A and B alike
          mma_bf16_16816(acc[m][f], xlo.x, xhi.x, xlo.y, xhi.y, wv[u][f].x, wv[u][f].y);
          mma_bf16_16816(acc[m][f], xlo.z, xhi.z, xlo.w, xhi.w, wv[u][f].z, wv[u][f].w);
        }
      }
    }
  }

  // fold the eight warps' partial sums: 4-7 into 0-3, 2-3 into 0-1, 1 into 0
#pragma unroll 1
  for (int half = kSkWarps / 2; half >= 1; half >>= 1) {
    if (warp >= half && warp < 2 * half) {
      float* dst = red + (size_t)(warp - half) * R * 32 + lane;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int f = 0; f < 4; ++f)
#pragma unroll
          for (int r = 0; r < 4; ++r) dst[((m * 4 + f) * 4 + r) * 32] = acc[m][f][r];
    }
    __syncthreads();
    if (warp < half) {
      const float* src = red + (size_t)warp * R * 32 + lane;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int f = 0; f < 4; ++f)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[m][f][r] += src[((m * 4 + f) * 4 + r) * 32];
    }
    __syncthreads();
  }
  if (warp != 0) return;

  const int splits = gridDim.y;
  if (splits > 1) {
    float* mine = ws + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * (R * 32) + lane;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int f = 0; f < 4; ++f)
#pragma unroll
        for (int r = 0; r < 4; ++r) mine[((m * 4 + f) * 4 + r) * 32] = acc[m][f][r];
    __threadfence();
    __syncwarp();
    unsigned prev = 0;
    if (lane == 0) prev = atomicAdd(counters + blockIdx.x, 1u);
    prev = __shfl_sync(0xffffffffu, prev, 0);
    if (prev != unsigned(splits - 1)) return;   // not the last CTA of this column group
    __threadfence();
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int f = 0; f < 4; ++f)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[m][f][r] = 0.f;
    for (int s = 0; s < splits; ++s) {   // every part from the workspace, in index order: the sum is the same whoever is last
      const float* part = ws + ((size_t)s * gridDim.x + blockIdx.x) * (R * 32) + lane;
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int f = 0; f < 4; ++f)
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[m][f][r] += __ldcg(part + ((m * 4 + f) * 4 + r) * 32);
    }
    if (lane == 0) counters[blockIdx.x] = 0u;   // ready for the next launch on this stream
  }

#pragma unroll
  for (int m = 0; m < MT; ++m) {
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const int col = n0 + f * 8 + q * 2;
      if (col >= N) continue;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = m * 16 + g + h * 8;
        if (row >= M) continue;
        float v0 = acc[m][f][h * 2], v1 = acc[m][f][h * 2 + 1];
        if (residual) {
          const float2 rv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(residual + (long long)row * ldr + col));
          v0 += rv.x;
          v1 += rv.y;
        }
        *reinterpret_cast<uint32_t*>(y + (long long)row * ldy + col) = pack_bf16x2(v0, v1);
      }
    }
  }
}

struct SkinnyWs {
  float* ws = nullptr;
  unsigned* counters = nullptr;
};
static std::mutex g_sk_mu;
// Measured under graph replay (Llama-1.1B shapes, 32 and 128 rows): the hand-over of partial sums through L2 costs about 3 us, more
// than a 2048-deep K loop on a third of the SMs, so by default K is split only when a warp still keeps 16 chunks (K >= 8192).
static std::atomic<int> g_sk_target{1};       // CTAs per SM the K split aims for (lt_gemm_skinny_set_target)
static std::atomic<int> g_sk_min_chunks{16};  // 32-element chunks a warp keeps at least when K is split
static std::map<std::pair<int, cudaStream_t>, SkinnyWs> g_sk_ws;

// Workspace of the K split, one per (device, stream): launches on one stream are serialised and the last CTA of a
// column group resets its counter.  Not allocated while the stream records a graph (the launch then runs unsplit).
static bool get_skinny_ws(cudaStream_t st, SkinnyWs* out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(g_sk_mu);
  auto key = std::make_pair(dev, st);
  auto it = g_sk_ws.find(key);
  if (it != g_sk_ws.end()) { *out = it->second; return out->ws != nullptr; }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return false;
  }
  void* base = nullptr;
  if (cudaMalloc(&base, kSkWsBytes + kSkCounters * sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    g_sk_ws[key] = SkinnyWs{};
    return false;
  }
  SkinnyWs w;
  w.ws = static_cast<float*>(base);
  w.counters = reinterpret_cast<unsigned*>(static_cast<char*>(base) + kSkWsBytes);
  if (cudaMemsetAsync(w.counters, 0, kSkCounters * sizeof(unsigned), st) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(base);
    g_sk_ws[key] = SkinnyWs{};
    return false;
  }
  g_sk_ws[key] = w;
  *out = w;
  return true;
}

template <int MT>
static int launch_skinny(const __nv_bfloat16* X, long long ldx, const __nv_bfloat16* W, long long ldw, __nv_bfloat16* Y, long long ldy,
                         const __nv_bfloat16* R, long long ldr, int M, int N, int K, cudaStream_t st) {
  static bool configured = false;
  constexpr int smem = 4 * MT * 16 * 32 * 4;
  auto kern = gemm_skinny_kernel<MT>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  const int sms = sm_count();
  const int groups = (N + kSkCols - 1) / kSkCols;
  const int nchunks = K / 32;
  int splits = (g_sk_target.load() * sms + groups - 1) / groups;
  const int mc = g_sk_min_chunks.load();
  const int max_splits = nchunks / (mc * kSkWarps) > 1 ? nchunks / (mc * kSkWarps) : 1;   // at least `mc` chunks per warp
  if (splits > max_splits) splits = max_splits;
  SkinnyWs wsp;
  if (splits > 1) {
    const size_t need = size_t(splits) * groups * (MT * 16 * 32) * sizeof(float);
    if (groups > kSkCounters || need > kSkWsBytes || !get_skinny_ws(st, &wsp)) splits = 1;
  }
  int per = (nchunks + splits - 1) / splits;
  splits = (nchunks + per - 1) / per;
  dim3 grid(groups, splits);
  kern<<<grid, kSkWarps * 32, smem, st>>>(X, ldx, W, ldw, Y, ldy, R, ldr, M, N, K, per, wsp.ws, wsp.counters);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // namespace lt

extern "C" {

// How many CTAs per SM the K split of narrow outputs aims for (default 1; 1 to 8) and how many 32-element chunks of K a
// warp keeps at least (default 16; 1 to 16).
int lt_gemm_skinny_set_target(int ctas_per_sm, int min_chunks_per_warp) {
  lt::g_sk_target.store(ctas_per_sm < 1 ? 1 : (ctas_per_sm > 8 ? 8 : ctas_per_sm));
  lt::g_sk_min_chunks.store(min_chunks_per_warp < 1 ? 1 : (min_chunks_per_warp > 16 ? 16 : min_chunks_per_warp));
  return 0;
}

// y[M, N] = x[M, K] @ w[N, K]^T (+ residual[M, N]), all bf16; 1 <= M <= 128, K a multiple of 32, N a multiple of 8, operand
// rows 16-byte aligned, y / residual rows 4-byte aligned.
int lt_gemm_skinny_bf16(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy, const void* residual,
                        long long ldr, int M, int N, int K, void* stream) {
  using namespace lt;
  if (M < 1 || M > 128 || N <= 0 || K <= 0 || (K & 31) || (N & 7) || (ldx & 7) || (ldw & 7) || (ldy & 1) || (ldr & 1) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(y) & 3) ||
      (reinterpret_cast<uintptr_t>(residual) & 3))
    return -int(kStatusBadArgument);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  if (M <= 16) return launch_skinny<1>(X, ldx, W, ldw, Y, ldy, R, ldr, M, N, K, st);
  if (M <= 32) return launch_skinny<2>(X, ldx, W, ldw, Y, ldy, R, ldr, M, N, K, st);
  if (M <= 64) return launch_skinny<4>(X, ldx, W, ldw, Y, ldy, R, ldr, M, N, K, st);
  return launch_skinny<8>(X, ldx, W, ldw, Y, ldy, R, ldr, M, N, K, st);
}

}  // extern "C"
