// Cross-entropy (vocab-parallel capable, backward fused in place) and the optimizer kernels.
//
// Reference counterparts: cross_entropy_loss_forward/backward, one thread per row and a serial loop over
// the vocabulary (src/backend/gpu_native/nn/nn_kernels.cu:1070-1116); adamw_step_kernel launched once per
// parameter tensor (src/backend/gpu_native/optim/optimizers.cu:3-124); GradScaler's inf check through
// Ops::max(Ops::abs(g)) (src/optim/grad_scaler.cpp:29-33); host-side clip_grad_norm_ (src/ops/clip_grad.cpp:8-52).
//
// Here: a CTA per row with an online (max, sum-exp) scan; the statistics of a vocabulary shard are
// exposed so that tensor-parallel ranks can combine them with one tiny collective before the in-place
// gradient pass; AdamW/Adam/SGD/RMSprop run over flat buffers or over a pointer table in ONE launch,
// with the gradient unscale and the skip-on-overflow decision read from device memory.
#include "lt_cuda.h"
#include <cuda_fp8.h>

#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kCeThreads = 256;

__device__ __forceinline__ void ce_ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// stats[row] = {max, sum exp(l - max), target logit if the target falls in [vocab_start, vocab_start+V) else 0}
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ targets,
                int vocab_start, int N, int V, float* __restrict__ stats, int vec_ok) {
  __shared__ float sm[32], ss[32];
  for (int row = blockIdx.x; row < N; row += gridDim.x) {
    const __nv_bfloat16* lr = logits + (long long)row * ldl;
    float m = -INFINITY, s = 0.f;
    const int v8 = vec_ok ? V / 8 : 0;
    for (int i = threadIdx.x; i < v8; i += blockDim.x) {
      float f[8];
      ce_ld8(lr + i * 8, f);
      float cm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
      const float nm = fmaxf(m, cm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int i = v8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
      const float f = __bfloat162float(lr[i]);
      const float nm = fmaxf(m, f);
      s = s * __expf(m - nm) + __expf(f - nm);
      m = nm;
    }
    // combine (m, s) across the block
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { sm[warp] = m; ss[warp] = s; }
    __syncthreads();
    if (warp == 0) {
      m = (lane < (blockDim.x >> 5)) ? sm[lane] : -INFINITY;
      s = (lane < (blockDim.x >> 5)) ? ss[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, m, o);
        const float os = __shfl_xor_sync(0xffffffffu, s, o);
        const float nm = fmaxf(m, om);
        s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
        m = nm;
      }
      if (lane == 0) {
        const long long t = targets[row] - vocab_start;
        stats[row * 3 + 0] = m;
        stats[row * 3 + 1] = s;
        stats[row * 3 + 2] = (t >= 0 && t < V) ? __bfloat162float(lr[t]) : 0.f;
      }
    }
  }
}

// gstats[row] = {global max, global sum-exp, target logit}.  loss[row] = log(sum) + max - target (0 if ignored);
// logits are overwritten by dlogits = (softmax - onehot) * grad_scale when write_grad != 0.
__global__ void __launch_bounds__(kCeThreads)
ce_finish_kernel(__nv_bfloat16* __restrict__ logits, long long ldl, const long long* __restrict__ targets,
                 int vocab_start, int N, int V, const float* __restrict__ gstats, float* __restrict__ loss,
                 float grad_scale, long long ignore_index, int write_grad, int vec_ok) {
  for (int row = blockIdx.x; row < N; row += gridDim.x) {
    __nv_bfloat16* lr = logits + (long long)row * ldl;
    const long long tgt = targets[row];
    const bool ignored = (tgt == ignore_index);
    const float gm = gstats[row * 3 + 0], gs = gstats[row * 3 + 1], gt = gstats[row * 3 + 2];
    if (threadIdx.x == 0 && loss) loss[row] = ignored ? 0.f : (__logf(gs) + gm - gt);
    if (!write_grad) continue;
    const float inv = ignored ? 0.f : grad_scale / gs;
    const long long t = tgt - vocab_start;
    const int v8 = vec_ok ? V / 8 : 0;
    for (int i = threadIdx.x; i < v8; i += blockDim.x) {
      float f[8];
      ce_ld8(lr + i * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = __expf(f[j] - gm) * inv;
        if (!ignored && (long long)(i * 8 + j) == t) g -= grad_scale;
        f[j] = g;
      }
      uint4 u;
      u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
      u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
      *reinterpret_cast<uint4*>(lr + i * 8) = u;
    }
    for (int i = v8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
      float g = __expf(__bfloat162float(lr[i]) - gm) * inv;
      if (!ignored && (long long)i == t) g -= grad_scale;
      lr[i] = __float2bfloat16(g);
    }
  }
}

// ---------------------------------------------------------------------------------------------- optimizers
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;  // bc = 1 - beta^t
  int adamw;                                  // 1 decoupled weight decay, 0 L2 (Adam)
};

__device__ __forceinline__ float adam_update(float p, float g, float& m, float& v, const AdamArgs& a) {
  if (!a.adamw) g += a.wd * p;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float mh = m / a.bc1, vh = v / a.bc2;
  if (a.adamw) p -= a.lr * a.wd * p;
  return p - a.lr * mh / (sqrtf(vh) + a.eps);
}

// dyn (nullable, device): dyn[0] = multiplier applied to every gradient, dyn[1] != 0 -> skip the step.
template <typename GradT>
__global__ void adam_flat_kernel(float* __restrict__ master, const GradT* __restrict__ grad, float* __restrict__ m,
                                 float* __restrict__ v, __nv_bfloat16* __restrict__ param_bf16, long long n,
                                 AdamArgs a, const float* __restrict__ dyn) {
  float gmul = 1.f;
  if (dyn) {
    if (dyn[1] != 0.f) return;
    gmul = dyn[0];
  }
  // 4 elements per thread per step (16-byte accesses of the fp32 arrays), scalar tail
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    if (sizeof(GradT) == 2) {
      const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(grad) + i * 4);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      const float4 u = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad) + i * 4);
      g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
    }
    float4 p4 = *reinterpret_cast<const float4*>(master + i * 4);
    float4 m4 = *reinterpret_cast<const float4*>(m + i * 4);
    float4 v4 = *reinterpret_cast<const float4*>(v + i * 4);
    float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) pp[j] = adam_update(pp[j], g[j] * gmul, mm[j], vv[j], a);
    *reinterpret_cast<float4*>(master + i * 4) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(m + i * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *reinterpret_cast<float4*>(v + i * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (param_bf16) {
      uint2 o;
      o.x = pack_bf16x2(pp[0], pp[1]);
      o.y = pack_bf16x2(pp[2], pp[3]);
      *reinterpret_cast<uint2*>(param_bf16 + i * 4) = o;
    }
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g;
    if (sizeof(GradT) == 2) g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[i]);
    else g = reinterpret_cast<const float*>(grad)[i];
    g *= gmul;
    float mm = m[i], vv = v[i];
    const float p = adam_update(master[i], g, mm, vv, a);
    m[i] = mm; v[i] = vv; master[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16(p);
  }
}

// Pointer-table variant: chunk c covers elements [chunk_off[c], +chunk_len) of tensor chunk_tensor[c].
// Tensor t has fp32 param p[t], grad g[t] (fp32 or bf16 by gdtype[t]), m[t], v[t], optional bf16 copy.
struct TensorTable {
  float* const* p;
  const void* const* g;
  float* const* m;
  float* const* v;
  __nv_bfloat16* const* p16;
  const long long* numel;
  const int* g_is_bf16;
  const int* chunk_tensor;
  const long long* chunk_off;
};
constexpr int kChunk = 65536;

__global__ void adam_table_kernel(TensorTable tb, int n_chunks, AdamArgs a, const float* __restrict__ dyn) {
  float gmul = 1.f;
  if (dyn) {
    if (dyn[1] != 0.f) return;
    gmul = dyn[0];
  }
  for (int c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    const int t = tb.chunk_tensor[c];
    const long long off = tb.chunk_off[c];
    const long long end = min(off + (long long)kChunk, tb.numel[t]);
    float* p = tb.p[t];
    float* m = tb.m[t];
    float* v = tb.v[t];
    __nv_bfloat16* p16 = tb.p16 ? tb.p16[t] : nullptr;
    const bool gb = tb.g_is_bf16[t] != 0;
    // 4 elements per thread per step where every array is 16-byte aligned (chunk offsets are multiples of 4, so this is
    // a property of the tensors' base addresses); the scalar loop below takes the tail, or everything otherwise
    long long done_to = off;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                           (reinterpret_cast<uintptr_t>(tb.g[t]) << (gb ? 1 : 0)) |
                           (p16 ? (reinterpret_cast<uintptr_t>(p16) << 1) : 0);
    if ((bits & 15u) == 0) {
      const long long n4 = (end - off) / 4;
      for (long long q = threadIdx.x; q < n4; q += blockDim.x) {
        const long long i = off + q * 4;
        float g[4];
        if (gb) {
          const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(tb.g[t]) + i);
          const float2 a0 = unpack_bf16x2(u.x), a1 = unpack_bf16x2(u.y);
          g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y;
        } else {
          const float4 u = *reinterpret_cast<const float4*>(static_cast<const float*>(tb.g[t]) + i);
          g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
        }
        const float4 p4 = *reinterpret_cast<const float4*>(p + i);
        const float4 m4 = *reinterpret_cast<const float4*>(m + i);
        const float4 v4 = *reinterpret_cast<const float4*>(v + i);
        float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) pp[j] = adam_update(pp[j], g[j] * gmul, mm[j], vv[j], a);
        *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
        *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
        *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        if (p16) {
          uint2 o;
          o.x = pack_bf16x2(pp[0], pp[1]);
          o.y = pack_bf16x2(pp[2], pp[3]);
          *reinterpret_cast<uint2*>(p16 + i) = o;
        }
      }
      done_to = off + n4 * 4;
    }
    for (long long i = done_to + threadIdx.x; i < end; i += blockDim.x) {
      float g = gb ? __bfloat162float(static_cast<const __nv_bfloat16*>(tb.g[t])[i]) : static_cast<const float*>(tb.g[t])[i];
      g *= gmul;
      float mm = m[i], vv = v[i];
      const float np = adam_update(p[i], g, mm, vv, a);
      m[i] = mm; v[i] = vv; p[i] = np;
      if (p16) p16[i] = __float2bfloat16(np);
    }
  }
}

// SGD with momentum / RMSprop over a flat fp32 buffer.
__global__ void sgd_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ vel, long long n,
                                float lr, float momentum, float wd) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gg = g[i] + wd * p[i];
    if (vel) {
      const float nv = momentum * vel[i] + gg;
      vel[i] = nv;
      gg = nv;
    }
    p[i] -= lr * gg;
  }
}
__global__ void rmsprop_flat_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ sq, long long n,
                                    float lr, float alpha, float eps, float wd) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gg = g[i] + wd * p[i];
    const float s = alpha * sq[i] + (1.f - alpha) * gg * gg;
    sq[i] = s;
    p[i] -= lr * gg / (sqrtf(s) + eps);
  }
}


// ---------------------------------------------------------------------------------------------- AdamW, 8-bit moments
// m and v are stored as int8 codes (one absmax scale per tensor: value = code * scale, scale = absmax / 127) or as
// e4m3 codes (delayed scaling: scale = max of the last ten absmax values / 240).  Reference: AdamW8bit / AdamWFP8
// (src/optim/adamw_8bit.cpp:13-104, src/optim/adamw_fp8.cpp:13-126), CPU loops there.  Here one step of one tensor
// is three launches and no host synchronisation: pass 0 computes the updated moments only to find their absmax
// (atomicMax on the float's bit pattern), a one-thread kernel turns the absmax into the new scales (and keeps the
// e4m3 history), pass 1 recomputes the moments, updates the parameter and stores the codes with the new scales.
struct AdamQArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;
  int fp8, first, p_bf16, g_bf16;
};
__device__ __forceinline__ float ldf(const void* base, int is_bf16, long long i) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(base)[i]) : static_cast<const float*>(base)[i];
}
__device__ __forceinline__ float deq8(const void* q, int fp8, long long i, float scale) {
  if (fp8) return float(static_cast<const __nv_fp8_e4m3*>(q)[i]) * scale;
  return float(static_cast<const signed char*>(q)[i]) * scale;
}
__global__ void adam_q_kernel(void* __restrict__ p, const void* __restrict__ g, void* __restrict__ mq, void* __restrict__ vq,
                              long long n, AdamQArgs a, const float* __restrict__ scale_old, const float* __restrict__ scale_new,
                              unsigned* __restrict__ amax, int pass) {
  const float so_m = scale_old[0], so_v = scale_old[1];
  float sn_m = 1.f, sn_v = 1.f;
  if (pass == 1) { sn_m = scale_new[0]; sn_v = scale_new[1]; }
  float am = 0.f, av = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gg = ldf(g, a.g_bf16, i);
    const float m0 = a.first ? 0.f : deq8(mq, a.fp8, i, so_m);
    const float v0 = a.first ? 0.f : deq8(vq, a.fp8, i, so_v);
    const float m = a.beta1 * m0 + (1.f - a.beta1) * gg;
    const float v = a.beta2 * v0 + (1.f - a.beta2) * gg * gg;
    if (pass == 0) {
      am = fmaxf(am, fabsf(m));
      av = fmaxf(av, fabsf(v));
      continue;
    }
    float w = ldf(p, a.p_bf16, i);
    w -= a.lr * a.wd * w;
    w -= a.lr * (m / a.bc1) / (sqrtf(v / a.bc2) + a.eps);
    if (a.p_bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(w);
    else static_cast<float*>(p)[i] = w;
    if (a.fp8) {
      static_cast<__nv_fp8_e4m3*>(mq)[i] = __nv_fp8_e4m3(fminf(fmaxf(m / sn_m, -448.f), 448.f));
      static_cast<__nv_fp8_e4m3*>(vq)[i] = __nv_fp8_e4m3(fminf(fmaxf(v / sn_v, -448.f), 448.f));
    } else {
      static_cast<signed char*>(mq)[i] = (signed char)fminf(fmaxf(rintf(m / sn_m), -127.f), 127.f);
      static_cast<signed char*>(vq)[i] = (signed char)fminf(fmaxf(rintf(v / sn_v), -127.f), 127.f);
    }
  }
  if (pass == 0) {
    for (int o = 16; o > 0; o >>= 1) {
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
      av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, o));
    }
    if ((threadIdx.x & 31) == 0) {               // non-negative floats order like their bit patterns
      atomicMax(amax, __float_as_uint(am));
      atomicMax(amax + 1, __float_as_uint(av));
    }
  }
}
// state: [0..1] absmax of this step (bit patterns, cleared here), hist: [2][10] floats, hist_n: steps recorded so far.
__global__ void adam_q_scales_kernel(unsigned* __restrict__ amax, float* __restrict__ scale_new, float* __restrict__ hist,
                                     int* __restrict__ hist_n, int fp8) {
  if (threadIdx.x >= 2) return;
  const int k = threadIdx.x;
  const float a = __uint_as_float(amax[k]);
  amax[k] = 0u;
  float s;
  if (fp8) {
    const int nrec = *hist_n;
    hist[k * 10 + nrec % 10] = a;
    const int have = nrec + 1 < 10 ? nrec + 1 : 10;
    float mx = 0.f;
    for (int j = 0; j < have; ++j) mx = fmaxf(mx, hist[k * 10 + j]);
    s = mx > 0.f ? mx / 240.f : 1.f;
  } else {
    s = a > 0.f ? a / 127.f : 1.f;
  }
  scale_new[k] = s;
  __syncwarp(0x3u);
  if (k == 0 && fp8) *hist_n += 1;
}

// out[0] += sum x^2, out[1] += number of non-finite elements.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f, bad = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float f;
    if (sizeof(T) == 2) f = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]);
    else f = reinterpret_cast<const float*>(x)[i];
    if (!isfinite(f)) bad += 1.f; else s += f * f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    bad += __shfl_xor_sync(0xffffffffu, bad, o);
  }
  __shared__ float rs[32], rb[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { rs[warp] = s; rb[warp] = bad; }
  __syncthreads();
  if (warp == 0) {
    s = lane < (blockDim.x >> 5) ? rs[lane] : 0.f;
    bad = lane < (blockDim.x >> 5) ? rb[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      bad += __shfl_xor_sync(0xffffffffu, bad, o);
    }
    if (lane == 0) {
      atomicAdd(out, s);
      if (bad != 0.f) atomicAdd(out + 1, bad);
    }
  }
}

// dyn[0] = clip coefficient * inv_scale, dyn[1] = overflow flag, from stats = {sumsq, nonfinite}.
__global__ void clip_coef_kernel(const float* __restrict__ stats, float* __restrict__ dyn, float max_norm, float inv_scale) {
  const float norm = sqrtf(stats[0]) * inv_scale;
  float coef = 1.f;
  if (max_norm > 0.f && norm > max_norm) coef = max_norm / (norm + 1e-6f);
  dyn[0] = coef * inv_scale;
  dyn[1] = stats[1] != 0.f ? 1.f : 0.f;
  dyn[2] = norm;
}

inline int flat_grid(long long n) {
  long long g = (n + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  return int(g > cap ? cap : (g < 1 ? 1 : g));
}

}  // namespace lt

extern "C" {

int lt_ce_stats(const void* logits, long long ldl, const long long* targets, int vocab_start, int N, int V, float* stats,
                void* stream) {
  using namespace lt;
  if (N == 0) return 0;
  const int vec_ok = (ldl % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int grid = N < sm_count() * 8 ? N : sm_count() * 8;
  ce_stats_kernel<<<grid, kCeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ldl, targets, vocab_start, N, V, stats, vec_ok);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_ce_finish(void* logits, long long ldl, const long long* targets, int vocab_start, int N, int V, const float* gstats,
                 float* loss, float grad_scale, long long ignore_index, int write_grad, void* stream) {
  using namespace lt;
  if (N == 0) return 0;
  const int vec_ok = (ldl % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  const int grid = N < sm_count() * 8 ? N : sm_count() * 8;
  ce_finish_kernel<<<grid, kCeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ldl, targets, vocab_start, N, V, gstats, loss, grad_scale, ignore_index, write_grad, vec_ok);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_adam_flat(float* master, const void* grad, int grad_is_bf16, float* m, float* v, void* param_bf16, long long n,
                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, int adamw,
                 const float* dyn, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, adamw};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (grad_is_bf16)
    adam_flat_kernel<__nv_bfloat16><<<flat_grid(n), 256, 0, st>>>(master, static_cast<const __nv_bfloat16*>(grad), m, v,
                                                                 static_cast<__nv_bfloat16*>(param_bf16), n, a, dyn);
  else
    adam_flat_kernel<float><<<flat_grid(n), 256, 0, st>>>(master, static_cast<const float*>(grad), m, v,
                                                         static_cast<__nv_bfloat16*>(param_bf16), n, a, dyn);
  LT_LAUNCH_CHECK();
  return 0;
}

// All table pointers are device arrays prepared by the caller (n_tensors / n_chunks entries).
int lt_adam_table(const void* p_ptrs, const void* g_ptrs, const void* m_ptrs, const void* v_ptrs, const void* p16_ptrs,
                  const long long* numel, const int* g_is_bf16, const int* chunk_tensor, const long long* chunk_off,
                  int n_chunks, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, int adamw,
                  const float* dyn, void* stream) {
  using namespace lt;
  if (n_chunks == 0) return 0;
  TensorTable tb{static_cast<float* const*>(p_ptrs), static_cast<const void* const*>(g_ptrs),
                 static_cast<float* const*>(m_ptrs), static_cast<float* const*>(v_ptrs),
                 static_cast<__nv_bfloat16* const*>(p16_ptrs), numel, g_is_bf16, chunk_tensor, chunk_off};
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, adamw};
  const int cap = sm_count() * 8;
  adam_table_kernel<<<n_chunks < cap ? n_chunks : cap, 256, 0, static_cast<cudaStream_t>(stream)>>>(tb, n_chunks, a, dyn);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_adam_chunk_elems() { return lt::kChunk; }

// One AdamW step of one tensor whose moments are int8 (fp8 = 0) or e4m3 (fp8 = 1) codes.  scale_old / scale_new: two
// floats each (m, v); amax: two uint32, zero before the first step; hist: 20 floats, hist_n: one int (both zero at
// the start; used by the e4m3 variant).  first != 0: the moments do not exist yet (treated as zero).
int lt_adam_q8(void* p, int p_bf16, const void* g, int g_bf16, void* mq, void* vq, long long n, float lr, float beta1, float beta2,
               float eps, float wd, float bc1, float bc2, int fp8, int first, const float* scale_old, float* scale_new,
               void* amax, float* hist, int* hist_n, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  AdamQArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, fp8, first, p_bf16, g_bf16};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  adam_q_kernel<<<flat_grid(n), 256, 0, st>>>(p, g, mq, vq, n, a, scale_old, scale_new, static_cast<unsigned*>(amax), 0);
  adam_q_scales_kernel<<<1, 32, 0, st>>>(static_cast<unsigned*>(amax), scale_new, hist, hist_n, fp8);
  adam_q_kernel<<<flat_grid(n), 256, 0, st>>>(p, g, mq, vq, n, a, scale_old, scale_new, static_cast<unsigned*>(amax), 1);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_sgd_flat(float* p, const float* g, float* vel, long long n, float lr, float momentum, float wd, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  sgd_flat_kernel<<<flat_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, g, vel, n, lr, momentum, wd);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_rmsprop_flat(float* p, const float* g, float* sq, long long n, float lr, float alpha, float eps, float wd, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  rmsprop_flat_kernel<<<flat_grid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, g, sq, n, lr, alpha, eps, wd);
  LT_LAUNCH_CHECK();
  return 0;
}
// out: 2 floats, accumulated into (zero them before the first call of a step).
int lt_sumsq(const void* x, int is_bf16, long long n, float* out, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<flat_grid(n), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  else sumsq_kernel<float><<<flat_grid(n), 256, 0, st>>>(static_cast<const float*>(x), n, out);
  LT_LAUNCH_CHECK();
  return 0;
}
// dyn: 3 floats {grad multiplier, overflow flag, grad norm}.
int lt_clip_coef(const float* stats, float* dyn, float max_norm, float inv_scale, void* stream) {
  lt::clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(stats, dyn, max_norm, inv_scale);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
