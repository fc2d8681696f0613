// Paged-KV decode attention (one query token per sequence) with split-K, grouped-query heads and bf16 or
// e4m3 KV caches, plus the KV-append kernel that fills the cache.
//
// Reference: paged_attention_forward runs one THREAD per (sequence, head) with a 2048-float local score
// array and float block tables (src/backend/gpu_native/nn/nn_kernels.cu:1256-1312), flash-decoding exists
// only on the CPU (src/ops/flash_decoding.cpp:13-115), and nothing writes the cache.  Here a warp owns one
// (sequence, query head, split): lanes span the head dimension, keys stream through an online softmax, and a
// second kernel merges the per-split (max, sum, partial output) triples.  Decode is bandwidth bound (each
// K/V byte is used once per query head of its group), so the kernel is plain CUDA-core code.
// Cache layout: [num_blocks, Hkv, block_size, D] as in the reference.
#include <cuda_fp8.h>

#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

template <int D, bool FP8>
__device__ __forceinline__ void load_row(const void* base, long long elem_off, int lane, float (&out)[D / 32]) {
  constexpr int E = D / 32;
  if (FP8) {
    const __nv_fp8_e4m3* p = static_cast<const __nv_fp8_e4m3*>(base) + elem_off + lane * E;
#pragma unroll
    for (int i = 0; i < E; ++i) out[i] = float(p[i]);
  } else {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(base) + elem_off + lane * E;
#pragma unroll
    for (int i = 0; i < E; i += 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
      out[i] = f.x;
      out[i + 1] = f.y;
    }
  }
}

// part: [S, Hq, splits, D + 2] fp32 = (partial output normalised by its own sum, max, sum)
template <int D, bool FP8>
__global__ void paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const void* __restrict__ k_cache,
                                    const void* __restrict__ v_cache, const int* __restrict__ block_tables,
                                    const int* __restrict__ context_lens, float* __restrict__ part, int S, int Hq, int Hkv,
                                    int block_size, int max_blocks, int splits, float scale, float k_scale, float v_scale) {
  constexpr int E = D / 32;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = S * Hq * splits;
  if (warp_global >= total) return;
  const int sp = warp_global % splits;
  const int h = (warp_global / splits) % Hq;
  const int s = warp_global / (splits * Hq);
  const int hkv = h / (Hq / Hkv);
  const int ctx = context_lens[s];
  const int per = (ctx + splits - 1) / splits;
  const int t0 = sp * per, t1 = min(ctx, t0 + per);
  float qv[E];
  {
    const __nv_bfloat16* qp = q + ((long long)s * Hq + h) * D + lane * E;
#pragma unroll
    for (int i = 0; i < E; ++i) qv[i] = __bfloat162float(qp[i]) * scale * k_scale;
  }
  float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  for (int t = t0; t < t1; ++t) {
    const int blk = block_tables[(long long)s * max_blocks + t / block_size];
    const long long off = (((long long)blk * Hkv + hkv) * block_size + (t % block_size)) * D;
    float kv[E];
    load_row<D, FP8>(k_cache, off, lane, kv);
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) d += qv[i] * kv[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    const float nm = fmaxf(m, d);
    const float a = __expf(m - nm), p = __expf(d - nm);
    load_row<D, FP8>(v_cache, off, lane, kv);
    l = l * a + p;
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] = acc[i] * a + p * kv[i];
    m = nm;
  }
  float* out = part + (((long long)s * Hq + h) * splits + sp) * (D + 2);
  const float inv = l > 0.f ? v_scale / l : 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) out[lane * E + i] = acc[i] * inv;
  if (lane == 0) { out[D] = m; out[D + 1] = l; }
}


// ---------------------------------------------------------------------------------------------- grouped-query decode
// One CTA of four warps owns one (sequence, KV head, split): every K / V byte of its key range is read once for the
// whole group of G = Hq / Hkv query heads (the warp-per-query-head kernel above reads it G times and walks the keys
// one at a time).  A warp takes 32 keys at a time:
//   scores   lane = key: the lane reads its key row with 16-byte loads (the 32 rows of a chunk are contiguous in a
//            cache block) and forms the dot products with the G query vectors, which sit in shared memory pre-scaled
//            (all lanes read the same address: a broadcast);
//   softmax  per head, one max and one sum reduction per 32 keys; running (max, sum) kept per warp;
//   P V      lane = pair (D 64) or quad (D 128) of output columns: the probabilities of the chunk go through shared
//            memory, then for each key the warp reads the V row as one coalesced line and every lane updates its G x E
//            accumulators.
// The warps' partial results are merged in shared memory and written in the (normalised output, max, sum) form that
// the merge kernel above already combines across splits.  bf16 caches only (e4m3 stays on the kernel above).
constexpr int kPdWarps = 4;
constexpr int kPdMaxG = 8;

template <int D>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_gqa_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables,
                        const int* __restrict__ context_lens, float* __restrict__ part, int S, int Hq, int Hkv, int block_size,
                        int max_blocks, int splits, float scale) {
  constexpr int E = D / 32;
  const int G = Hq / Hkv;
  const int sp = blockIdx.x % splits;
  const int hkv = (blockIdx.x / splits) % Hkv;
  const int s = blockIdx.x / (splits * Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ float q_s[kPdMaxG][D];
  __shared__ float p_s[kPdWarps][32][kPdMaxG];            // [warp][key of the chunk][head]
  __shared__ float red_m[kPdWarps][kPdMaxG], red_l[kPdWarps][kPdMaxG];
  __shared__ float red_o[kPdWarps][kPdMaxG][D];
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    q_s[g][d] = __bfloat162float(q[((long long)s * Hq + hkv * G + g) * D + d]) * scale;
  }
  __syncthreads();
  const int ctx = context_lens[s];
  const int per = ((ctx + splits - 1) / splits + 31) / 32 * 32;      // whole 32-key chunks per split
  const int t0 = sp * per, t1 = min(ctx, t0 + per);
  float m[kPdMaxG], l[kPdMaxG], acc[kPdMaxG][E];
#pragma unroll
  for (int g = 0; g < kPdMaxG; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }
  const int* bt = block_tables + (long long)s * max_blocks;
  for (int c0 = t0 + warp * 32; c0 < t1; c0 += kPdWarps * 32) {
    // ---- scores of this lane's key for every head of the group
    const int t = c0 + lane;
    const bool live = t < t1;
    float sc[kPdMaxG];
#pragma unroll
    for (int g = 0; g < kPdMaxG; ++g) sc[g] = 0.f;
    int my_blk = 0, my_off = 0;
    if (live) {
      my_blk = bt[t / block_size];
      my_off = t % block_size;
      const uint4* kr = reinterpret_cast<const uint4*>(k_cache + (((long long)my_blk * Hkv + hkv) * block_size + my_off) * D);
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        const uint4 u = kr[j];
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
#pragma unroll
        for (int g = 0; g < kPdMaxG; ++g) {
          if (g < G) {
            const float4 q0 = *reinterpret_cast<const float4*>(&q_s[g][j * 8]);
            const float4 q1 = *reinterpret_cast<const float4*>(&q_s[g][j * 8 + 4]);
            sc[g] += a.x * q0.x + a.y * q0.y + b.x * q0.z + b.y * q0.w + c.x * q1.x + c.y * q1.y + d.x * q1.z + d.y * q1.w;
          }
        }
      }
    }
    // ---- online softmax per head over the 32 keys of the chunk
#pragma unroll
    for (int g = 0; g < kPdMaxG; ++g) {
      if (g < G) {
        float mx = live ? sc[g] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float nm = fmaxf(m[g], mx);
        const float a = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - nm);
        const float pv = live ? __expf(sc[g] - nm) : 0.f;
        float ps = pv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l[g] = l[g] * a + ps;
        m[g] = nm;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] *= a;
        p_s[warp][lane][g] = pv;
      } else {
        p_s[warp][lane][g] = 0.f;
      }
    }
    __syncwarp();
    // ---- P V: lane = E output columns; one coalesced V row per key.  U rows are requested before the first is used,
    // so a warp keeps U x D x 2 bytes in flight instead of one row (a single row per warp left the kernel bound by
    // memory latency at a tenth of the copy bandwidth).
    constexpr int U = (D == 64) ? 16 : 8;
    const int nk = min(32, t1 - c0);
#pragma unroll 1
    for (int kk0 = 0; kk0 < nk; kk0 += U) {
      float vv[U][E];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int kk = kk0 + u;
        const int blk_u = __shfl_sync(0xffffffffu, my_blk, kk & 31);
        const int off_u = __shfl_sync(0xffffffffu, my_off, kk & 31);
        if (kk < nk) {
          const __nv_bfloat16* vr = v_cache + (((long long)blk_u * Hkv + hkv) * block_size + off_u) * D + lane * E;
          if (E == 2) {
            const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(vr));
            vv[u][0] = f.x; vv[u][1] = f.y;
          } else {
            const uint2 w2 = *reinterpret_cast<const uint2*>(vr);
            const float2 f0 = unpack_bf16x2(w2.x), f1 = unpack_bf16x2(w2.y);
            vv[u][0] = f0.x; vv[u][1] = f0.y; vv[u][E - 2] = f1.x; vv[u][E - 1] = f1.y;
          }
        } else {
#pragma unroll
          for (int e = 0; e < E; ++e) vv[u][e] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int kk = (kk0 + u) & 31;                  // rows beyond nk carry zeros (and their probabilities are zero)
        const float4 p0 = *reinterpret_cast<const float4*>(&p_s[warp][kk][0]);
        const float4 p1 = *reinterpret_cast<const float4*>(&p_s[warp][kk][4]);
        const float pg[kPdMaxG] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int g = 0; g < kPdMaxG; ++g)
          if (g < G) {
#pragma unroll
            for (int e = 0; e < E; ++e) acc[g][e] += pg[g] * vv[u][e];
          }
      }
    }
    __syncwarp();
  }
  // ---- merge the four warps, write this split's partial result
#pragma unroll
  for (int g = 0; g < kPdMaxG; ++g)
    if (g < G) {
      if (lane == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
#pragma unroll
      for (int e = 0; e < E; ++e) red_o[warp][g][lane * E + e] = acc[g][e];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) gm = fmaxf(gm, red_m[w][g]);
    float lsum = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
      if (red_m[w][g] == -INFINITY) continue;
      const float a = __expf(red_m[w][g] - gm);
      lsum += red_l[w][g] * a;
      o += red_o[w][g][d] * a;
    }
    float* out = part + (((long long)s * Hq + hkv * G + g) * splits + sp) * (D + 2);
    out[d] = lsum > 0.f ? o / lsum : 0.f;
    if (d == 0) { out[D] = gm; out[D + 1] = lsum; }
  }
}

template <int D>
__global__ void paged_decode_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ o, int rows, int splits) {
  const int row = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  constexpr int E = D / 32;
  float gm = -INFINITY;
  for (int sp = 0; sp < splits; ++sp) gm = fmaxf(gm, part[((long long)row * splits + sp) * (D + 2) + D]);
  float wsum = 0.f, acc[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc[i] = 0.f;
  for (int sp = 0; sp < splits; ++sp) {
    const float* p = part + ((long long)row * splits + sp) * (D + 2);
    const float l = p[D + 1];
    if (l <= 0.f) continue;
    const float w = l * __expf(p[D] - gm);
    wsum += w;
#pragma unroll
    for (int i = 0; i < E; ++i) acc[i] += w * p[lane * E + i];
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) o[(long long)row * D + lane * E + i] = __float2bfloat16(acc[i] * inv);
}

// slot = block * block_size + offset for each new token.
template <bool FP8>
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                 void* __restrict__ k_cache, void* __restrict__ v_cache, const int* __restrict__ slots,
                                 long long n_tok, int Hkv, int D, int block_size, float k_inv_scale, float v_inv_scale) {
  const long long total = n_tok * Hkv * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int d = int(i % D);
    const int h = int((i / D) % Hkv);
    const long long t = i / ((long long)D * Hkv);
    const int slot = slots[t];
    if (slot < 0) continue;
    const long long dst = (((long long)(slot / block_size) * Hkv + h) * block_size + (slot % block_size)) * D + d;
    if (FP8) {
      static_cast<__nv_fp8_e4m3*>(k_cache)[dst] = __nv_fp8_e4m3(__bfloat162float(k_new[i]) * k_inv_scale);
      static_cast<__nv_fp8_e4m3*>(v_cache)[dst] = __nv_fp8_e4m3(__bfloat162float(v_new[i]) * v_inv_scale);
    } else {
      static_cast<__nv_bfloat16*>(k_cache)[dst] = k_new[i];
      static_cast<__nv_bfloat16*>(v_cache)[dst] = v_new[i];
    }
  }
}

}  // namespace lt

extern "C" {

// q: [S, Hq, D] bf16; caches [num_blocks, Hkv, block_size, D] bf16 (kv_fp8 = 0) or e4m3 (kv_fp8 = 1, with the
// dequantisation scales k_scale / v_scale); block_tables [S, max_blocks] int32; context_lens [S] int32;
// part: scratch [S, Hq, splits, D + 2] fp32; o: [S, Hq, D] bf16.
int lt_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables, const int* context_lens,
                    float* part, void* o, int S, int Hq, int Hkv, int D, int block_size, int max_blocks, int splits,
                    float scale, int kv_fp8, float k_scale, float v_scale, void* stream) {
  using namespace lt;
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || splits < 1) return -int(kStatusBadArgument);
  if (S == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int warps = S * Hq * splits;
  const int threads = 128;
  const int blocks = (warps * 32 + threads - 1) / threads;
  auto Q = static_cast<const __nv_bfloat16*>(q);
#define LT_PD(DD, F8) \
  paged_decode_kernel<DD, F8><<<blocks, threads, 0, st>>>(Q, k_cache, v_cache, block_tables, context_lens, part, S, Hq, Hkv, \
                                                          block_size, max_blocks, splits, scale, k_scale, v_scale)
  const int G = Hq / Hkv;
  if (!kv_fp8 && G <= kPdMaxG && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0) {
    // bf16 caches: every K / V byte is read once for the whole group of query heads
    const int ctas = S * Hkv * splits;
    auto KC = static_cast<const __nv_bfloat16*>(k_cache);
    auto VC = static_cast<const __nv_bfloat16*>(v_cache);
    if (D == 64) paged_decode_gqa_kernel<64><<<ctas, kPdWarps * 32, 0, st>>>(Q, KC, VC, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale);
    else paged_decode_gqa_kernel<128><<<ctas, kPdWarps * 32, 0, st>>>(Q, KC, VC, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale);
  } else if (D == 64) { if (kv_fp8) LT_PD(64, true); else LT_PD(64, false); }
  else { if (kv_fp8) LT_PD(128, true); else LT_PD(128, false); }
#undef LT_PD
  LT_LAUNCH_CHECK();
  const int rows = S * Hq;
  const int mb = (rows + 3) / 4;
  if (D == 64) paged_decode_merge_kernel<64><<<mb, 128, 0, st>>>(part, static_cast<__nv_bfloat16*>(o), rows, splits);
  else paged_decode_merge_kernel<128><<<mb, 128, 0, st>>>(part, static_cast<__nv_bfloat16*>(o), rows, splits);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int* slots, long long n_tok, int Hkv,
                 int D, int block_size, int kv_fp8, float k_scale, float v_scale, void* stream) {
  using namespace lt;
  if (n_tok == 0) return 0;
  const long long total = n_tok * Hkv * D;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto KN = static_cast<const __nv_bfloat16*>(k_new);
  auto VN = static_cast<const __nv_bfloat16*>(v_new);
  if (kv_fp8) kv_append_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(KN, VN, k_cache, v_cache, slots, n_tok, Hkv, D, block_size, 1.f / k_scale, 1.f / v_scale);
  else kv_append_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(KN, VN, k_cache, v_cache, slots, n_tok, Hkv, D, block_size, 1.f, 1.f);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
