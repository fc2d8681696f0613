// Memory-bound bf16 kernels of the transformer block: RoPE (interleaved pairs), SwiGLU, GELU(tanh),
// residual add, embedding gather / scatter-add, dtype casts, fills.
//
// Reference counterparts: rope_forward/backward (src/backend/gpu_native/nn/nn_kernels.cu:1204-1254),
// gelu_forward/backward (:1118-1146), embedding_forward/backward (:1148-1188), elementwise family
// (src/backend/gpu_native/elementwise/elementwise_ops.cu:3-98), cast kernels (:362-430).
// The reference has no SiLU/SwiGLU; it is added because the Llama-style configurations need it.
// Every kernel moves 16 bytes per thread per access and grid-strides.
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---------------------------------------------------------------------------------------------- RoPE
// In-place rotation of `heads` heads of width `hd` inside rows of pitch `row_stride` (elements).
// Row r belongs to position (r % T) + pos_offset... positions are given explicitly when pos != nullptr.
// Pair convention: (x[2i], x[2i+1]) rotated by angle pos * theta^(-2i/hd)  (interleaved, as the reference).
// cos/sin tables are [max_pos, hd/2] fp32. sign = +1 forward, -1 backward (inverse rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, long long rows, int T,
                            int heads, int hd, long long row_stride, float sign) {
  const int vec_per_head = hd / 8;
  const long long total = rows * heads * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = int(i % vec_per_head);
    const int h = int((i / vec_per_head) % heads);
    const long long r = i / ((long long)vec_per_head * heads);
    const int t = pos ? pos[r] : int(r % T);
    __nv_bfloat16* p = x + r * row_stride + (long long)h * hd + v * 8;
    float f[8];
    ld8(p, f);
    const float4 c4 = *reinterpret_cast<const float4*>(cos_t + (long long)t * (hd / 2) + v * 4);
    const float4 s4 = *reinterpret_cast<const float4*>(sin_t + (long long)t * (hd / 2) + v * 4);
    const float c[4] = {c4.x, c4.y, c4.z, c4.w};
    const float s[4] = {s4.x * sign, s4.y * sign, s4.z * sign, s4.w * sign};
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = f[2 * j] * c[j] - f[2 * j + 1] * s[j];
      o[2 * j + 1] = f[2 * j] * s[j] + f[2 * j + 1] * c[j];
    }
    st8(p, o);
  }
}

// ---------------------------------------------------------------------------------------------- SwiGLU
// gu: [M, 2F] with gate in columns [0,F) and up in [F,2F).  h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long M, int F) {
  const int vpr = F / 8;
  const long long total = M * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = int(i % vpr) * 8;
    float g[8], u[8], o[8];
    ld8(gu + r * 2 * F + c, g);
    ld8(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    st8(h + r * F + c, o);
  }
}
// dgu may alias gu (written in place).
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* gu, const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* dgu,
                                  long long M, int F) {
  const int vpr = F / 8;
  const long long total = M * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = int(i % vpr) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + r * 2 * F + c, g);
    ld8(gu + r * 2 * F + F + c, u);
    ld8(dh + r * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
    }
    st8(dgu + r * 2 * F + c, dg);
    st8(dgu + r * 2 * F + F + c, du);
  }
}

// ---------------------------------------------------------------------------------------------- GELU / add / scale
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    ld8(x + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = gelu_tanh(f[j]);
    st8(y + i * 8, f);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    ld8(x + i * 8, f);
    ld8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      const float xx = f[j];
      const float t = tanhf(k0 * (xx + k1 * xx * xx * xx));
      const float dt = (1.f - t * t) * k0 * (1.f + 3.f * k1 * xx * xx);
      g[j] *= 0.5f * (1.f + t) + 0.5f * xx * dt;
    }
    st8(dx + i * 8, g);
  }
}
// out = a * alpha + b * beta  (b may be null)
__global__ void axpby_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out, float alpha, float beta, long long n8) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    ld8(a + i * 8, f);
    if (b) {
      float g[8];
      ld8(b + i * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * alpha + g[j] * beta;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= alpha;
    }
    st8(out + i * 8, f);
  }
}

// ---------------------------------------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long n_tok, int D, int V) {
  const int vpr = D / 8;
  const long long total = n_tok * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = int(i % vpr) * 8;
    long long t = idx[r];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    *reinterpret_cast<uint4*>(out + r * D + c) = __ldg(reinterpret_cast<const uint4*>(table + t * D + c));
  }
}
// dtable[idx[r]] += dout[r]   (bf16x2 atomics; dtable must be zeroed or hold the running gradient)
__global__ void embedding_bwd_kernel(const long long* __restrict__ idx, const __nv_bfloat16* __restrict__ dout,
                                     __nv_bfloat16* __restrict__ dtable, long long n_tok, int D, int V) {
  const int ppr = D / 2;
  const long long total = n_tok * ppr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ppr;
    const int c = int(i % ppr) * 2;
    long long t = idx[r];
    if (t < 0 || t >= V) continue;
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dout + r * D + c);
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + t * D + c), v);
  }
}

// ---------------------------------------------------------------------------------------------- casts / fills
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  const long long n8 = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const float4 a = *reinterpret_cast<const float4*>(in + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(in + i * 8 + 4);
    uint4 u;
    u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w);
    u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint4*>(out + i * 8) = u;
  }
  const long long tail = n8 * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = __float2bfloat16(in[tail]);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long n) {
  const long long n8 = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    ld8(in + i * 8, f);
    *reinterpret_cast<float4*>(out + i * 8) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  const long long tail = n8 * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tail < n) out[tail] = __bfloat162float(in[tail]);
}

inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return int(g);
}

}  // namespace lt

extern "C" {

int lt_rope(void* x, const float* cos_t, const float* sin_t, const int* pos, long long rows, int T, int heads, int hd,
            long long row_stride, int backward, void* stream) {
  using namespace lt;
  if (hd % 8 != 0 || row_stride % 8 != 0) return -int(kStatusBadArgument);
  const long long work = rows * heads * (hd / 8);
  if (work == 0) return 0;
  rope_kernel<<<grid_for(work, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), cos_t, sin_t, pos, rows, T, heads, hd, row_stride, backward ? -1.f : 1.f);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_swiglu_fwd(const void* gu, void* h, long long M, int F, void* stream) {
  using namespace lt;
  if (F % 8 != 0) return -int(kStatusBadArgument);
  if (M == 0) return 0;
  swiglu_fwd_kernel<<<grid_for(M * (F / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(h), M, F);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long M, int F, void* stream) {
  using namespace lt;
  if (F % 8 != 0) return -int(kStatusBadArgument);
  if (M == 0) return 0;
  swiglu_bwd_kernel<<<grid_for(M * (F / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dh), static_cast<__nv_bfloat16*>(dgu), M, F);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  using namespace lt;
  if (n % 8 != 0) return -int(kStatusBadArgument);
  if (n == 0) return 0;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n / 8);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream) {
  using namespace lt;
  if (n % 8 != 0) return -int(kStatusBadArgument);
  if (n == 0) return 0;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), n / 8);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_axpby(const void* a, const void* b, void* out, float alpha, float beta, long long n, void* stream) {
  using namespace lt;
  if (n % 8 != 0) return -int(kStatusBadArgument);
  if (n == 0) return 0;
  axpby_kernel<<<grid_for(n / 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(out), alpha, beta, n / 8);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_embedding_fwd(const long long* idx, const void* table, void* out, long long n_tok, int D, int V, void* stream) {
  using namespace lt;
  if (D % 8 != 0) return -int(kStatusBadArgument);
  if (n_tok == 0) return 0;
  embedding_fwd_kernel<<<grid_for(n_tok * (D / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), n_tok, D, V);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_embedding_bwd(const long long* idx, const void* dout, void* dtable, long long n_tok, int D, int V, void* stream) {
  using namespace lt;
  if (D % 2 != 0) return -int(kStatusBadArgument);
  if (n_tok == 0) return 0;
  embedding_bwd_kernel<<<grid_for(n_tok * (D / 2), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dtable), n_tok, D, V);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_cast_f32_to_bf16(const float* in, void* out, long long n, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n / 8 + 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, static_cast<__nv_bfloat16*>(out), n);
  LT_LAUNCH_CHECK();
  return 0;
}
int lt_cast_bf16_to_f32(const void* in, float* out, long long n, void* stream) {
  using namespace lt;
  if (n == 0) return 0;
  cast_bf16_to_f32_kernel<<<grid_for(n / 8 + 8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(in), out, n);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
