// Smaller sm_100a kernels that complete the op inventory:
//   * mixture-of-experts router: fp32 softmax over the experts, top-k, renormalisation, per-expert token counts and
//     probability mass for the load-balancing loss, and its backward
//     (reference: src/ops/moe_ops.cpp:11-193 and moe_gate_kernel, src/backend/gpu_native/nn/nn_kernels.cu:1339-1422,
//     one thread per token there; one warp per token here),
//   * dropout with a counter-based Philox generator (reference: generate_dropout_mask, nn_kernels.cu:1190-1202, an LCG
//     hash), the same (seed, offset) regenerates the mask in backward, so no mask tensor is stored,
//   * row softmax forward / backward (reference: softmax_forward_kernel, nn_kernels.cu:631-675, one thread per row),
//   * e4m3 quantiser with one scale per 128 x 128 weight block,
//   * GradScaler step: unscale a flat gradient buffer and detect inf / nan in the same pass
//     (reference: python/litetorch/amp.py GradScaler.unscale_, a host loop),
//   * full sum / max reductions (reference: cub::DeviceReduce in math/reduction.cu:25-58),
//   * strided gather to a contiguous tensor (make_contiguous_kernel / cat_forward_kernel,
//     elementwise/elementwise_ops.cu:133-179, 432-502).
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"
#include <cuda_fp8.h>

namespace lt {

// ------------------------------------------------------------------------------------------------ router
constexpr int kRouterMaxE = 256;   // experts per token a warp can hold (8 per lane)
constexpr int kRouterMaxK = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits [N, E] (fp32 or bf16) -> probs [N, E] fp32 (full softmax, kept for backward and the auxiliary loss),
// topk_w [N, k] fp32 (renormalised when `renorm`), topk_idx [N, k] int32, counts [E] int32 (+= tokens routed),
// mass [E] fp32 (+= softmax probability of every token).
template <typename T>
__global__ void moe_router_kernel(const T* __restrict__ logits, float* __restrict__ probs, float* __restrict__ topk_w,
                                  int* __restrict__ topk_idx, int* __restrict__ counts, float* __restrict__ mass, int N, int E,
                                  int k, int renorm) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= N) return;
  float v[kRouterMaxE / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? float(logits[(long long)token * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) {
    const int e = i * 32 + lane;
    v[i] *= inv;
    if (e < E) {
      probs[(long long)token * E + e] = v[i];
      if (mass) atomicAdd(mass + e, v[i]);
    }
  }
  // top-k by k rounds of warp arg-max (ties go to the lower expert index)
  float wsel[kRouterMaxK];
  int isel[kRouterMaxK];
  float wsum = 0.f;
#pragma unroll
  for (int r = 0; r < kRouterMaxK; ++r) {
    if (r < k) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < kRouterMaxE / 32; ++i) {
        const int e = i * 32 + lane;
        if (e < E && (v[i] > best)) { best = v[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      wsel[r] = best; isel[r] = bi;
      wsum += best;
      if ((bi & 31) == lane) {   // taken
#pragma unroll
        for (int i = 0; i < kRouterMaxE / 32; ++i)
          if (i == (bi >> 5)) v[i] = -2.f;
      }
    }
  }
  if (lane == 0) {
    const float rn = renorm ? 1.f / fmaxf(wsum, 1e-20f) : 1.f;
#pragma unroll
    for (int r = 0; r < kRouterMaxK; ++r) {
      if (r < k) {
        topk_w[(long long)token * k + r] = wsel[r] * rn;
        topk_idx[(long long)token * k + r] = isel[r];
        if (counts) atomicAdd(counts + isel[r], 1);
      }
    }
  }
}

// dlogits [N, E] fp32 from d(topk_w) [N, k] and an optional dense d(probs) [N, E] (auxiliary loss).
// w_r = p_{i_r} / S (S = sum of the selected p when renorm, else 1):  dp_{i_r} += (dw_r - sum_j dw_j w_j) / S,
// then the softmax Jacobian: dlogit_e = p_e (dp_e - sum_j dp_j p_j).
__global__ void moe_router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topk_idx,
                                      const float* __restrict__ topk_w, const float* __restrict__ d_topk_w,
                                      const float* __restrict__ d_probs, float* __restrict__ dlogits, int N, int E, int k,
                                      int renorm) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= N) return;
  float pv[kRouterMaxE / 32], dp[kRouterMaxE / 32];
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) {
    const int e = i * 32 + lane;
    pv[i] = e < E ? probs[(long long)token * E + e] : 0.f;
    dp[i] = (e < E && d_probs) ? d_probs[(long long)token * E + e] : 0.f;
  }
  float dot = 0.f, S = 1.f;
  if (renorm) {
    S = 0.f;
    for (int r = 0; r < k; ++r) {
      const float w = topk_w[(long long)token * k + r];
      dot += d_topk_w[(long long)token * k + r] * w;
    }
    // S = p_{i_0} / w_0 for any selected expert with non-zero weight
    for (int r = 0; r < k; ++r) {
      const int idx = topk_idx[(long long)token * k + r];
      const float w = topk_w[(long long)token * k + r];
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < kRouterMaxE / 32; ++i)
        if (i == (idx >> 5)) mine = pv[i];
      const float p_sel = __shfl_sync(0xffffffffu, mine, idx & 31);
      if (w > 0.f && S == 0.f) S = p_sel / w;
    }
    if (S == 0.f) S = 1.f;
  }
  for (int r = 0; r < k; ++r) {
    const int idx = topk_idx[(long long)token * k + r];
    const float g = (d_topk_w[(long long)token * k + r] - dot) / S;
    if ((idx & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kRouterMaxE / 32; ++i)
        if (i == (idx >> 5)) dp[i] += g;
    }
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) s += dp[i] * pv[i];
  s = warp_sum(s);
#pragma unroll
  for (int i = 0; i < kRouterMaxE / 32; ++i) {
    const int e = i * 32 + lane;
    if (e < E) dlogits[(long long)token * E + e] = pv[i] * (dp[i] - s);
  }
}

// ------------------------------------------------------------------------------------------------ dropout (Philox)
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0; key.y += W1;
  }
  return ctr;
}

// y = x * keep / (1 - p) with keep ~ Bernoulli(1 - p); element i uses word (i & 3) of Philox counter (offset + i / 4).
// The same call with the upstream gradient as x is the backward pass.
template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p, unsigned long long seed,
                               unsigned long long offset) {
  const uint32_t thresh = p >= 1.f ? 0xFFFFFFFFu : uint32_t(double(p) * 4294967296.0);
  const float scale = p >= 1.f ? 0.f : 1.f / (1.f - p);
  const long long n4 = (n + 3) / 4;
  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < n4; g += (long long)gridDim.x * blockDim.x) {
    const unsigned long long c = offset + (unsigned long long)g;
    const uint4 rnd = philox4x32_10(make_uint4(uint32_t(c), uint32_t(c >> 32), 0u, 0u),
                                    make_uint2(uint32_t(seed), uint32_t(seed >> 32)));
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = g * 4 + j;
      if (i < n) y[i] = T(rr[j] >= thresh ? float(x[i]) * scale : 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------------------ softmax
// One warp per row of length D (any D; values are re-read from global memory in each of the three passes when the
// row does not fit 32 registers per lane).
template <typename T>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * D;
  float mx = -INFINITY;
  for (int c = lane; c < D; c += 32) mx = fmaxf(mx, float(xr[c]));
  mx = warp_max(mx);
  float sum = 0.f;
  for (int c = lane; c < D; c += 32) sum += __expf(float(xr[c]) - mx);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  T* yr = y + row * D;
  for (int c = lane; c < D; c += 32) yr[c] = T(__expf(float(xr[c]) - mx) * inv);
}

// dx = y * (dy - sum(dy * y))
template <typename T>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* yr = y + row * D;
  const T* gr = dy + row * D;
  float s = 0.f;
  for (int c = lane; c < D; c += 32) s += float(yr[c]) * float(gr[c]);
  s = warp_sum(s);
  T* dr = dx + row * D;
  for (int c = lane; c < D; c += 32) dr[c] = T(float(yr[c]) * (float(gr[c]) - s));
}

// ------------------------------------------------------------------------------------------------ 128 x 128 quantiser
// One CTA (256 threads) per 128 x 128 block of w [N, K] bf16: amax -> scale = amax / 448 -> e4m3 codes.
__global__ void __launch_bounds__(256) quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, long long ldw,
                                                            uint8_t* __restrict__ q, long long ldq, float* __restrict__ scales,
                                                            int N, int K) {
  __shared__ float red[8];
  __shared__ float scale_s;
  const int kb = blockIdx.x, nb = blockIdx.y;
  const int kblocks = gridDim.x;
  const int t = threadIdx.x;
  // thread t handles row (t / 2) + 0..., 64 columns: two threads per row
  const int r = nb * 128 + (t >> 1);
  const int c0 = kb * 128 + (t & 1) * 64;
  float vals[64];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (r < N && c0 + j * 8 + 7 < K) u = *reinterpret_cast<const uint4*>(w + (long long)r * ldw + c0 + j * 8);
    const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(uu[i]);
      vals[j * 8 + i * 2] = f.x; vals[j * 8 + i * 2 + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = warp_max(amax);
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  if (t == 0) {
    float a = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) a = fmaxf(a, red[i]);
    const float sc = fmaxf(a, 1e-12f) / 448.f;
    scale_s = sc;
    scales[(long long)nb * kblocks + kb] = sc;
  }
  __syncthreads();
  const float inv = 1.f / scale_s;
  if (r < N) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t pk[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int b0 = j * 16 + i * 4;
        uint16_t lo, hi;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(vals[b0 + 1] * inv), "f"(vals[b0] * inv));
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(vals[b0 + 3] * inv), "f"(vals[b0 + 2] * inv));
        pk[i] = uint32_t(lo) | (uint32_t(hi) << 16);
      }
      if (c0 + j * 16 + 15 < K)
        *reinterpret_cast<uint4*>(q + (long long)r * ldq + c0 + j * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ GradScaler step
// g *= inv_scale; *found_inf = 1 if any element was inf or nan before scaling.
template <typename T>
__global__ void unscale_check_kernel(T* __restrict__ g, long long n, float inv_scale, int* __restrict__ found_inf) {
  int bad = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = float(g[i]);
    if (!isfinite(v)) bad = 1;
    g[i] = T(v * inv_scale);
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicExch(found_inf, 1);
}

// ------------------------------------------------------------------------------------------------ reductions
// mode 0: sum, 1: max.  Stage 1: per-CTA partials; stage 2 (one CTA) folds them into out[0].
template <typename T>
__global__ void __launch_bounds__(256) reduce_stage1_kernel(const T* __restrict__ x, long long n, float* __restrict__ part,
                                                            int mode) {
  __shared__ float red[8];
  float acc = mode ? -INFINITY : 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = float(x[i]);
    acc = mode ? fmaxf(acc, v) : acc + v;
  }
  acc = mode ? warp_max(acc) : warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int i = 1; i < 8; ++i) a = mode ? fmaxf(a, red[i]) : a + red[i];
    part[blockIdx.x] = a;
  }
}
__global__ void __launch_bounds__(256) reduce_stage2_kernel(const float* __restrict__ part, int n, float* __restrict__ out,
                                                            int mode) {
  __shared__ float red[8];
  float acc = mode ? -INFINITY : 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc = mode ? fmaxf(acc, part[i]) : acc + part[i];
  acc = mode ? warp_max(acc) : warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = red[0];
    for (int i = 1; i < 8; ++i) a = mode ? fmaxf(a, red[i]) : a + red[i];
    out[0] = a;
  }
}

// ------------------------------------------------------------------------------------------------ strided copy
struct StridedDesc {
  long long shape[8];
  long long src_stride[8];   // in elements
  long long dst_stride[8];
  int ndim;
};
// dst[dst index] = src[src index] over an <= 8-D index space (make_contiguous, cat into a slice, permutes).
template <int BYTES>
__global__ void strided_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long n, StridedDesc d) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long rem = i, so = 0, dof = 0;
#pragma unroll
    for (int k = 7; k >= 0; --k) {
      if (k < d.ndim) {
        const long long idx = rem % d.shape[k];
        rem /= d.shape[k];
        so += idx * d.src_stride[k];
        dof += idx * d.dst_stride[k];
      }
    }
    if (BYTES == 2) reinterpret_cast<uint16_t*>(dst)[dof] = reinterpret_cast<const uint16_t*>(src)[so];
    else if (BYTES == 4) reinterpret_cast<uint32_t*>(dst)[dof] = reinterpret_cast<const uint32_t*>(src)[so];
    else if (BYTES == 8) reinterpret_cast<uint64_t*>(dst)[dof] = reinterpret_cast<const uint64_t*>(src)[so];
    else dst[dof] = src[so];
  }
}

static inline unsigned grid_for(long long n, int threads, int per_sm) {
  long long b = (n + threads - 1) / threads;
  const long long cap = (long long)sm_count() * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return unsigned(b);
}

// ------------------------------------------------------------------------------------------------ MoE expert backward, pointwise part
// One warp per routed slot.  From gu = [gate | up] (bf16 [S, 2F]), the unweighted gradient of the expert output's input
// dh_u (bf16 [S, F]) and the slot's gate weight w it produces, in one pass over the rows:
//   h = silu(gate) * up (rounded to bf16 as the forward stored it),
//   dw[s] = sum_f h * dh_u                  (gradient of the gate weight),
//   hw = h * w                              (A operand of the down-projection weight gradient),
//   dgu = SwiGLU backward of dh = dh_u * w  (input of the up-projection weight gradient and of dX).
// Padding slots (slot_src[s][0] < 0) write zeros and read nothing.
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16(x)); }

__global__ void moe_expert_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh_u,
                                      const float* __restrict__ w, const int* __restrict__ slot_src,
                                      __nv_bfloat16* __restrict__ dgu, __nv_bfloat16* __restrict__ hw,
                                      float* __restrict__ dw, int S, int F) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= S) return;
  const long long r = warp;
  const bool valid = slot_src[2 * r] >= 0;
  const float wr = valid ? w[r] : 0.f;
  float dot = 0.f;
  for (int c = lane * 8; c < F; c += 32 * 8) {
    uint4 og = make_uint4(0, 0, 0, 0), ou = og, oh = og;
    if (valid) {
      const uint4 g4 = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c);
      const uint4 u4 = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c);
      const uint4 d4 = *reinterpret_cast<const uint4*>(dh_u + r * F + c);
      const uint32_t gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
      uint32_t rg[4], ru[4], rh[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 g = unpack_bf16x2(gs[j]), u = unpack_bf16x2(us[j]), d = unpack_bf16x2(ds[j]);
        float dg[2], du[2], hh[2];
        const float gg[2] = {g.x, g.y}, uu[2] = {u.x, u.y}, dd[2] = {d.x, d.y};
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float sg = 1.f / (1.f + __expf(-gg[q]));
          const float silu = gg[q] * sg;
          const float h = round_bf16(silu * uu[q]);
          dot += h * dd[q];
          const float dh = round_bf16(dd[q] * wr);
          du[q] = dh * silu;
          dg[q] = dh * uu[q] * (sg + silu * (1.f - sg));
          hh[q] = h * wr;
        }
        rg[j] = pack_bf16x2(dg[0], dg[1]);
        ru[j] = pack_bf16x2(du[0], du[1]);
        rh[j] = pack_bf16x2(hh[0], hh[1]);
      }
      og = make_uint4(rg[0], rg[1], rg[2], rg[3]);
      ou = make_uint4(ru[0], ru[1], ru[2], ru[3]);
      oh = make_uint4(rh[0], rh[1], rh[2], rh[3]);
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + c) = og;
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + F + c) = ou;
    *reinterpret_cast<uint4*>(hw + r * F + c) = oh;
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[r] = dot;
}

}  // namespace lt

extern "C" {

// dtype: 0 = fp32, 1 = bf16 (logits).  counts / mass may be null.  E <= 256, k <= 8.
int lt_moe_router(const void* logits, int dtype, float* probs, float* topk_w, int* topk_idx, int* counts, float* mass, int N,
                  int E, int k, int renorm, void* stream) {
  using namespace lt;
  if (E < 1 || E > kRouterMaxE || k < 1 || k > kRouterMaxK || k > E) return -int(kStatusBadArgument);
  if (N <= 0) return 0;
  const int wpb = 8;
  const unsigned blocks = unsigned((N + wpb - 1) / wpb);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == 1)
    moe_router_kernel<__nv_bfloat16><<<blocks, wpb * 32, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), probs, topk_w,
                                                                   topk_idx, counts, mass, N, E, k, renorm);
  else
    moe_router_kernel<float><<<blocks, wpb * 32, 0, st>>>(static_cast<const float*>(logits), probs, topk_w, topk_idx, counts,
                                                           mass, N, E, k, renorm);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_moe_router_bwd(const float* probs, const int* topk_idx, const float* topk_w, const float* d_topk_w, const float* d_probs,
                      float* dlogits, int N, int E, int k, int renorm, void* stream) {
  using namespace lt;
  if (E < 1 || E > kRouterMaxE || k < 1 || k > kRouterMaxK) return -int(kStatusBadArgument);
  if (N <= 0) return 0;
  const int wpb = 8;
  moe_router_bwd_kernel<<<unsigned((N + wpb - 1) / wpb), wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      probs, topk_idx, topk_w, d_topk_w, d_probs, dlogits, N, E, k, renorm);
  LT_LAUNCH_CHECK();
  return 0;
}

// dtype: 0 = fp32, 1 = bf16.  Backward: call again with dy as x and the same (p, seed, offset).
int lt_dropout(const void* x, void* y, long long n, int dtype, float p, unsigned long long seed, unsigned long long offset,
               void* stream) {
  using namespace lt;
  if (n <= 0) return 0;
  if (p < 0.f || p > 1.f) return -int(kStatusBadArgument);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = grid_for((n + 3) / 4, 256, 8);
  if (dtype == 1)
    dropout_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y),
                                                          n, p, seed, offset);
  else
    dropout_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), n, p, seed, offset);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_softmax_fwd(const void* x, void* y, long long rows, int D, int dtype, void* stream) {
  using namespace lt;
  if (rows <= 0 || D <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = unsigned((rows + 7) / 8);
  if (dtype == 1)
    softmax_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                              static_cast<__nv_bfloat16*>(y), rows, D);
  else
    softmax_fwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), rows, D);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int D, int dtype, void* stream) {
  using namespace lt;
  if (rows <= 0 || D <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = unsigned((rows + 7) / 8);
  if (dtype == 1)
    softmax_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y),
                                                              static_cast<const __nv_bfloat16*>(dy),
                                                              static_cast<__nv_bfloat16*>(dx), rows, D);
  else
    softmax_bwd_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(y), static_cast<const float*>(dy),
                                                      static_cast<float*>(dx), rows, D);
  LT_LAUNCH_CHECK();
  return 0;
}

// w [N, K] bf16 (K a multiple of 128, ldw a multiple of 8) -> q [N, K] e4m3, scales [ceil(N/128), K/128] fp32.
int lt_quant_fp8_128x128(const void* w, long long ldw, void* q, long long ldq, float* scales, int N, int K, void* stream) {
  using namespace lt;
  if (N <= 0 || K <= 0) return 0;
  if (K % 128 != 0 || ldw % 8 != 0 || ldq % 16 != 0) return -int(kStatusBadArgument);
  dim3 grid(K / 128, (N + 127) / 128);
  quant_128x128_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(w), ldw,
                                                                            static_cast<uint8_t*>(q), ldq, scales, N, K);
  LT_LAUNCH_CHECK();
  return 0;
}

// dtype: 0 = fp32, 1 = bf16.  found_inf is a device int the caller zeroes before the first bucket of a step.
int lt_unscale_check(void* g, long long n, int dtype, float inv_scale, int* found_inf, void* stream) {
  using namespace lt;
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = grid_for(n, 256, 8);
  if (dtype == 1) unscale_check_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<__nv_bfloat16*>(g), n, inv_scale, found_inf);
  else            unscale_check_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(g), n, inv_scale, found_inf);
  LT_LAUNCH_CHECK();
  return 0;
}

// out[0] = sum (mode 0) or max (mode 1) of x[0..n); part: scratch of lt_reduce_parts() floats.
int lt_reduce_parts() { return lt::sm_count() * 4; }
int lt_reduce_all(const void* x, long long n, int dtype, int mode, float* part, float* out, void* stream) {
  using namespace lt;
  if (n <= 0) return -int(kStatusBadArgument);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = grid_for(n, 256, 4);
  if (dtype == 1) reduce_stage1_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, part, mode);
  else            reduce_stage1_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), n, part, mode);
  reduce_stage2_kernel<<<1, 256, 0, st>>>(part, int(blocks), out, mode);
  LT_LAUNCH_CHECK();
  return 0;
}

// Copy an <= 8-D index space: dst[sum idx*dst_stride] = src[sum idx*src_stride]; strides in elements of elem_bytes.
int lt_strided_copy(const void* src, void* dst, int ndim, const long long* shape, const long long* src_stride,
                    const long long* dst_stride, int elem_bytes, void* stream) {
  using namespace lt;
  if (ndim < 1 || ndim > 8) return -int(kStatusBadArgument);
  StridedDesc d{};
  long long n = 1;
  for (int i = 0; i < ndim; ++i) {
    d.shape[i] = shape[i]; d.src_stride[i] = src_stride[i]; d.dst_stride[i] = dst_stride[i];
    n *= shape[i];
  }
  d.ndim = ndim;
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = grid_for(n, 256, 8);
  auto s = static_cast<const uint8_t*>(src);
  auto t = static_cast<uint8_t*>(dst);
  switch (elem_bytes) {
    case 1: strided_copy_kernel<1><<<blocks, 256, 0, st>>>(s, t, n, d); break;
    case 2: strided_copy_kernel<2><<<blocks, 256, 0, st>>>(s, t, n, d); break;
    case 4: strided_copy_kernel<4><<<blocks, 256, 0, st>>>(s, t, n, d); break;
    case 8: strided_copy_kernel<8><<<blocks, 256, 0, st>>>(s, t, n, d); break;
    default: return -int(kStatusBadArgument);
  }
  LT_LAUNCH_CHECK();
  return 0;
}

// gu [S, 2F], dh_u [S, F] bf16; w [S] fp32; slot_src [S, 2] int32 (first column < 0: padding slot);
// dgu [S, 2F], hw [S, F] bf16 and dw [S] fp32 are written.  F must be a multiple of 8.
int lt_moe_expert_bwd(const void* gu, const void* dh_u, const void* w, const void* slot_src, void* dgu, void* hw, void* dw,
                      int S, int F, void* stream) {
  using namespace lt;
  if (S <= 0) return 0;
  if (F <= 0 || F % 8 != 0) return -int(kStatusBadArgument);
  const int threads = 256;
  const unsigned blocks = unsigned((S * 32ll + threads - 1) / threads);
  moe_expert_bwd_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh_u), static_cast<const float*>(w),
      static_cast<const int*>(slot_src), static_cast<__nv_bfloat16*>(dgu), static_cast<__nv_bfloat16*>(hw),
      static_cast<float*>(dw), S, F);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------- int8 quantisers
// Per-tensor: q = clamp(round(x / scale), -127, 127).  Per-row: scale[r] = absmax(row r) / 127 (1 for an all-zero row),
// a warp per row.  x is fp32 (is_bf16 = 0) or bf16.  Reference: include/litetorch/quantization.h:15-40 (CPU loops).
namespace lt {
__device__ __forceinline__ float ldq(const void* x, int is_bf16, long long i) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(x)[i]) : static_cast<const float*>(x)[i];
}
__global__ void quant_int8_tensor_kernel(const void* __restrict__ x, int is_bf16, signed char* __restrict__ q, long long n, float inv_scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    q[i] = (signed char)fminf(fmaxf(rintf(ldq(x, is_bf16, i) * inv_scale), -127.f), 127.f);
}
__global__ void quant_int8_rows_kernel(const void* __restrict__ x, int is_bf16, signed char* __restrict__ q, float* __restrict__ scale,
                                       int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const long long base = (long long)row * cols;
  float am = 0.f;
  for (int c = lane; c < cols; c += 32) am = fmaxf(am, fabsf(ldq(x, is_bf16, base + c)));
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float sc = am > 0.f ? am / 127.f : 1.f;
  if (lane == 0) scale[row] = sc;
  const float inv = 1.f / sc;
  for (int c = lane; c < cols; c += 32)
    q[base + c] = (signed char)fminf(fmaxf(rintf(ldq(x, is_bf16, base + c) * inv), -127.f), 127.f);
}
}  // namespace lt

namespace lt {
// Per-row e4m3 quantiser for the row-scaled fp8 GEMM (lt_gemm_e4m3): scale[r] = absmax(row r) / 448 (1 for an all-zero row),
// q = x / scale rounded to e4m3 with saturation.  A warp per row, 16 bytes per lane and step; cols a multiple of 8.
__global__ void quant_e4m3_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, __nv_fp8_e4m3* __restrict__ q, long long ldq,
                                       float* __restrict__ scale, int rows, int cols) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + (long long)row * ldx;
  float am = 0.f;
  for (int c = lane * 8; c < cols; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(w[i]);
      am = fmaxf(am, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float sc = am > 0.f ? am / 448.f : 1.f;
  if (lane == 0) scale[row] = sc;
  const float inv = 1.f / sc;
  __nv_fp8_e4m3* qr = q + (long long)row * ldq;
  for (int c = lane * 8; c < cols; c += 256) {
    const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    __nv_fp8_e4m3 o8[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = unpack_bf16x2(w[i]);
      o8[2 * i] = __nv_fp8_e4m3(f.x * inv);
      o8[2 * i + 1] = __nv_fp8_e4m3(f.y * inv);
    }
    *reinterpret_cast<uint2*>(qr + c) = *reinterpret_cast<const uint2*>(o8);
  }
}
}  // namespace lt

extern "C" {
// x [rows, cols] bf16 (pitch ldx elements, rows 16-byte aligned), q [rows, cols] e4m3 (pitch ldq bytes, rows 8-byte aligned),
// scale [rows] fp32.
int lt_quant_e4m3_rows(const void* x, long long ldx, void* q, long long ldq, float* scale, int rows, int cols, void* stream) {
  if (rows == 0 || cols == 0) return 0;
  if ((cols & 7) || (ldx & 7) || (ldq & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
    return -int(lt::kStatusBadArgument);
  lt::quant_e4m3_rows_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_fp8_e4m3*>(q), ldq, scale, rows, cols);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_quant_int8_tensor(const void* x, int is_bf16, void* q, long long n, float scale, void* stream) {
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  lt::quant_int8_tensor_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, is_bf16, static_cast<signed char*>(q), n, 1.f / scale);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_quant_int8_rows(const void* x, int is_bf16, void* q, float* scale, int rows, int cols, void* stream) {
  if (rows == 0 || cols == 0) return 0;
  lt::quant_int8_rows_kernel<<<(rows + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, is_bf16, static_cast<signed char*>(q), scale, rows, cols);
  LT_LAUNCH_CHECK();
  return 0;
}
}  // extern "C"
