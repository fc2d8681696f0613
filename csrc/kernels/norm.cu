// RMSNorm and LayerNorm, forward and fused backward, bf16 activations with fp32 math.
//
// The reference has LayerNorm only, one thread per row (src/backend/gpu_native/nn/nn_kernels.cu:677-808)
// and a fused add+LayerNorm forward (:711-744). Here a CTA owns a row (16-byte vector accesses, block
// reduction), an optional residual add is fused into the forward (the sum is written out for the next
// residual branch), and the backward produces dx in one pass while each CTA keeps partial dgamma/dbeta
// sums for the rows it visited; a second tiny kernel folds the partials.
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

#include <mutex>

namespace lt {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 t;
  t = unpack_bf16x2(u.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16x2(u.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16x2(u.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16x2(u.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// y = norm(x (+ res)) * w (+ b).  RMS: mean unused.  If sum_out != nullptr the pre-norm sum is stored.
template <bool kLayerNorm>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int M, int D, float eps) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (long long)row * D;
    const __nv_bfloat16* rr = res ? res + (long long)row * D : nullptr;
    __nv_bfloat16* sr = sum_out ? sum_out + (long long)row * D : nullptr;
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
      float f[8];
      load8(xr + c, f);
      if (rr) {
        float g[8];
        load8(rr + c, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        if (sr) {
          store8(sr + c, f);
          // keep exactly what later passes will read back
          load8(sr + c, f);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s1 += f[j]; s2 += f[j] * f[j]; }
    }
    float mean = 0.f;
    if (kLayerNorm) mean = block_sum(s1, red) / D;
    const float sq = block_sum(s2, red) / D;
    const float var = kLayerNorm ? fmaxf(sq - mean * mean, 0.f) : sq;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    const __nv_bfloat16* src = (rr && sr) ? sr : xr;
    for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
      float f[8], wv[8];
      load8(src + c, f);
      if (rr && !sr) {
        float g[8];
        load8(rr + c, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
      }
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * wv[j];
      if (b) {
        float bv[8];
        load8(b + c, bv);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += bv[j];
      }
      store8(y + (long long)row * D + c, f);
    }
  }
}

// dx (+= dres) and per-CTA partial dw/db.  ITERS = ceil(D / (threads*8)).
template <bool kLayerNorm, int ITERS>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part, float* __restrict__ db_part, int M, int D) {
  __shared__ float red[32];
  float dw_acc[ITERS][8], db_acc[ITERS][8];
#pragma unroll
  for (int i = 0; i < ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; }

  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const long long off = (long long)row * D;
    const float mean = kLayerNorm ? mean_in[row] : 0.f;
    const float rstd = rstd_in[row];
    float s_g = 0.f, s_gx = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = (i * kNormThreads + threadIdx.x) * 8;
      if (c < D) {
        float g[8], xv[8], wv[8];
        load8(dy + off + c, g);
        load8(x + off + c, xv);
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          dw_acc[i][j] += g[j] * xh;
          if (kLayerNorm) db_acc[i][j] += g[j];
          const float gw = g[j] * wv[j];
          s_g += gw;
          s_gx += gw * xh;
        }
      }
    }
    float m_g = 0.f;
    if (kLayerNorm) m_g = block_sum(s_g, red) / D;
    const float m_gx = block_sum(s_gx, red) / D;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = (i * kNormThreads + threadIdx.x) * 8;
      if (c < D) {
        float g[8], xv[8], wv[8], o[8];
        load8(dy + off + c, g);
        load8(x + off + c, xv);
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = (xv[j] - mean) * rstd;
          o[j] = rstd * (g[j] * wv[j] - m_g - xh * m_gx);
        }
        if (dres) {
          float r[8];
          load8(dres + off + c, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + off + c, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = (i * kNormThreads + threadIdx.x) * 8;
    if (c < D) {
      float* dwp = dw_part + (long long)blockIdx.x * D + c;
#pragma unroll
      for (int j = 0; j < 8; ++j) dwp[j] = dw_acc[i][j];
      if (kLayerNorm && db_part) {
        float* dbp = db_part + (long long)blockIdx.x * D + c;
#pragma unroll
        for (int j = 0; j < 8; ++j) dbp[j] = db_acc[i][j];
      }
    }
  }
}

// RMSNorm backward with ONE WARP PER ROW (D = 256 * ITERS, ITERS in {1, 2, 4, 8}): dy and x of the row stay in
// registers between the reduction and the dx pass, the row sums are warp shuffles (no block barrier per row), and a
// lane has 16 * ITERS bytes x 2 of loads in flight, so a CTA of 8 warps keeps 8 rows moving instead of one.
// dgamma is accumulated per lane over all rows of the warp and folded to one partial row per CTA at the end.
template <int ITERS>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                        const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                        float* __restrict__ dw_part, int M) {
  constexpr int D = 256 * ITERS;
  constexpr int kWarps = kNormThreads / 32;
  __shared__ float fold[kWarps][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float dw_acc[ITERS][8];
#pragma unroll
  for (int i = 0; i < ITERS; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dw_acc[i][j] = 0.f;

  for (int row = blockIdx.x * kWarps + warp; row < M; row += gridDim.x * kWarps) {
    const long long off = (long long)row * D;
    uint4 gq[ITERS], xq[ITERS];
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = (i * 32 + lane) * 8;
      gq[i] = *reinterpret_cast<const uint4*>(dy + off + c);
      xq[i] = *reinterpret_cast<const uint4*>(x + off + c);
    }
    const float rstd = rstd_in[row];
    float s_gx = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = (i * 32 + lane) * 8;
      float g[8], xv[8], wv[8];
      unpack8(gq[i], g);
      unpack8(xq[i], xv);
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = xv[j] * rstd;
        dw_acc[i][j] += g[j] * xh;
        s_gx += g[j] * wv[j] * xh;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s_gx += __shfl_xor_sync(0xffffffffu, s_gx, o);
    const float m_gx = s_gx / D;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int c = (i * 32 + lane) * 8;
      float g[8], xv[8], wv[8], o[8];
      unpack8(gq[i], g);
      unpack8(xq[i], xv);
      load8(w + c, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (g[j] * wv[j] - xv[j] * rstd * m_gx);
      if (dres) {
        float r[8];
        load8(dres + off + c, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      store8(dx + off + c, o);
    }
  }
  // one partial dgamma row per CTA: 256 columns at a time through shared memory
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) fold[warp][lane * 8 + j] = dw_acc[i][j];
    __syncthreads();
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < kWarps; ++k) sum += fold[k][threadIdx.x];
    dw_part[(long long)blockIdx.x * D + i * 256 + threadIdx.x] = sum;
    __syncthreads();
  }
}

// out[c] (+)= sum_p part[p, c]; out is bf16 or fp32.  A block owns 32 columns; its 8 warps split the partial rows.
__global__ void fold_partials_kernel(const float* __restrict__ part, void* __restrict__ out, int P, int D,
                                     int out_fp32, int accumulate) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < D)
    for (int p = w; p < P; p += 8) s += part[(long long)p * D + c];
  red[w][lane] = s;
  __syncthreads();
  if (w != 0 || c >= D) return;
#pragma unroll
  for (int i = 1; i < 8; ++i) s += red[i][lane];
  if (out_fp32) {
    float* o = static_cast<float*>(out);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

}  // namespace lt

extern "C" {

// Number of CTAs the backward uses; the caller sizes the partial buffers [ctas, D] fp32 with it.
int lt_norm_bwd_ctas(int M) {
  const int cap = lt::sm_count() * 2;
  return M < cap ? M : cap;
}

int lt_norm_fwd(int layer_norm, const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out,
                float* mean_out, float* rstd_out, int M, int D, float eps, void* stream) {
  using namespace lt;
  if (D % 8 != 0) return -int(kStatusBadArgument);
  if (M == 0) return 0;
  const int grid = M < sm_count() * 8 ? M : sm_count() * 8;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto S = static_cast<__nv_bfloat16*>(sum_out);
  if (layer_norm) norm_fwd_kernel<true><<<grid, kNormThreads, 0, st>>>(X, R, W, B, Y, S, mean_out, rstd_out, M, D, eps);
  else            norm_fwd_kernel<false><<<grid, kNormThreads, 0, st>>>(X, R, W, nullptr, Y, S, nullptr, rstd_out, M, D, eps);
  LT_LAUNCH_CHECK();
  return 0;
}

// dw_part/db_part: scratch [lt_norm_bwd_ctas(M), D] fp32. dw/db: bf16 or fp32 [D].
int lt_norm_bwd(int layer_norm, const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                const void* dres, void* dx, float* dw_part, float* db_part, void* dw, void* db, int grads_fp32,
                int accumulate, int M, int D, void* stream) {
  using namespace lt;
  if (D % 8 != 0 || D > kNormThreads * 8 * 8) return -int(kStatusBadArgument);
  if (M == 0) return 0;
  const int grid = lt_norm_bwd_ctas(M);
  const int iters = (D + kNormThreads * 8 - 1) / (kNormThreads * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  if (!layer_norm && (D == 256 || D == 512 || D == 1024 || D == 2048) && M >= 8 * grid / 2) {
    // warp-per-row kernel; grid CTAs of 8 warps, one partial dgamma row per CTA
    int g2 = (M + 7) / 8;
    if (g2 > grid) g2 = grid;
    if (g2 > sm_count()) g2 = sm_count();
    switch (D) {
      case 256: rmsnorm_bwd_warp_kernel<1><<<g2, kNormThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_part, M); break;
      case 512: rmsnorm_bwd_warp_kernel<2><<<g2, kNormThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_part, M); break;
      case 1024: rmsnorm_bwd_warp_kernel<4><<<g2, kNormThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_part, M); break;
      default: rmsnorm_bwd_warp_kernel<8><<<g2, kNormThreads, 0, st>>>(DY, X, W, rstd, DR, DX, dw_part, M); break;
    }
    LT_LAUNCH_CHECK();
    fold_partials_kernel<<<(D + 31) / 32, 256, 0, st>>>(dw_part, dw, g2, D, grads_fp32, accumulate);
    LT_LAUNCH_CHECK();
    return 0;
  }
#define LT_NORM_BWD(LN, IT) \
  norm_bwd_kernel<LN, IT><<<grid, kNormThreads, 0, st>>>(DY, X, W, mean, rstd, DR, DX, dw_part, db_part, M, D)
  if (layer_norm) {
    if (iters <= 1) LT_NORM_BWD(true, 1); else if (iters <= 2) LT_NORM_BWD(true, 2);
    else if (iters <= 4) LT_NORM_BWD(true, 4); else LT_NORM_BWD(true, 8);
  } else {
    if (iters <= 1) LT_NORM_BWD(false, 1); else if (iters <= 2) LT_NORM_BWD(false, 2);
    else if (iters <= 4) LT_NORM_BWD(false, 4); else LT_NORM_BWD(false, 8);
  }
#undef LT_NORM_BWD
  LT_LAUNCH_CHECK();
  const int fb = (D + 31) / 32;
  fold_partials_kernel<<<fb, 256, 0, st>>>(dw_part, dw, grid, D, grads_fp32, accumulate);
  if (layer_norm && db && db_part) fold_partials_kernel<<<fb, 256, 0, st>>>(db_part, db, grid, D, grads_fp32, accumulate);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in norm_noalloc.h).
// ------------------------------------------------------------------------------------------------
#include <atomic>
#include <initializer_list>
#include "norm_noalloc.h"

namespace lt {
// Partial dgamma / dbeta sums: [2][LT_NORM_NOALLOC_MAX_CTAS][LT_NORM_NOALLOC_MAX_D] fp32.
static __device__ __align__(256) float g_norm_noalloc_scratch[2 * LT_NORM_NOALLOC_MAX_CTAS * LT_NORM_NOALLOC_MAX_D];

// In host code the array's name is only a handle; the device address has to be looked up, once per device,
// with that device current.
static float* norm_noalloc_scratch_ptr(int* err) {
  static std::atomic<float*> ptrs[64];    // zero-initialised; published with release, read with acquire
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *err = LT_NORM_NOALLOC_ERR_SETUP; return nullptr; }
  if (float* known = ptrs[dev].load(std::memory_order_acquire)) return known;
  std::lock_guard<std::mutex> lk(mu);
  if (float* known = ptrs[dev].load(std::memory_order_acquire)) return known;
  float* p = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_noalloc_scratch);
  if (e != cudaSuccess || p == nullptr) { *err = LT_NORM_NOALLOC_ERR_SETUP; return nullptr; }
  ptrs[dev].store(p, std::memory_order_release);
  return p;
}
}  // namespace lt

extern "C" int lt_norm_bwd_noalloc(int layer_norm, const void* dy, const void* x, const void* w, const float* mean,
                                   const float* rstd, const void* dres, void* dx, void* dw, void* db, int grads_fp32,
                                   int accumulate, int M, int D, void* stream) {
  using namespace lt;
  if (D % 8 != 0 || D <= 0 || M < 0) return -int(kStatusBadArgument);
  if (D > LT_NORM_NOALLOC_MAX_D) return LT_NORM_NOALLOC_ERR_TOO_LARGE;
  if (M == 0) return 0;
  // Nothing is launched on a missing or misaligned pointer: the kernels use 16-byte accesses on every row, and a
  // bad address on the device would be a memory fault instead of an error code.
  if (!dy || !x || !w || !rstd || !dx || !dw || (layer_norm && (!mean || !db))) return -int(kStatusBadArgument);
  for (const void* q : {dy, x, w, static_cast<const void*>(dx), dres})
    if (q && (reinterpret_cast<uintptr_t>(q) & 15u) != 0) return -int(kStatusBadArgument);
  for (const void* q : {static_cast<const void*>(mean), static_cast<const void*>(rstd), static_cast<const void*>(dw),
                        static_cast<const void*>(db)})
    if (q && (reinterpret_cast<uintptr_t>(q) & 3u) != 0) return -int(kStatusBadArgument);
  int err = 0;
  float* scratch = norm_noalloc_scratch_ptr(&err);
  if (!scratch) return err;
  float* dw_part = scratch;
  float* db_part = scratch + (size_t)LT_NORM_NOALLOC_MAX_CTAS * LT_NORM_NOALLOC_MAX_D;
  const int grid = M < LT_NORM_NOALLOC_MAX_CTAS ? M : LT_NORM_NOALLOC_MAX_CTAS;
  const int iters = (D + kNormThreads * 8 - 1) / (kNormThreads * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
#define LT_NORM_BWD_NA(LN, IT) \
  norm_bwd_kernel<LN, IT><<<grid, kNormThreads, 0, st>>>(DY, X, W, mean, rstd, DR, DX, dw_part, db_part, M, D)
  if (layer_norm) {
    if (iters <= 1) LT_NORM_BWD_NA(true, 1); else LT_NORM_BWD_NA(true, 2);
  } else {
    if (iters <= 1) LT_NORM_BWD_NA(false, 1); else LT_NORM_BWD_NA(false, 2);
  }
#undef LT_NORM_BWD_NA
  LT_LAUNCH_CHECK();
  const int fb = (D + 31) / 32;
  fold_partials_kernel<<<fb, 256, 0, st>>>(dw_part, dw, grid, D, grads_fp32, accumulate);
  if (layer_norm && db) fold_partials_kernel<<<fb, 256, 0, st>>>(db_part, db, grid, D, grads_fp32, accumulate);
  LT_LAUNCH_CHECK();
  return 0;
}
