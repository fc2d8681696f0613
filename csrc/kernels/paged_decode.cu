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
#include "lt_cuda.h"
#include <cuda_fp8.h>

#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

// Plain (non-multicast) bulk asynchronous copy global -> this CTA's shared memory; bytes a multiple of 16, both
// addresses 16-byte aligned; completion is counted on the mbarrier.
__device__ __forceinline__ void bulk_g2s_pd(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}

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
// one at a time).  A warp takes 32 keys at a time, and the K and V rows of the chunks ahead are already on their way:
//   loads    the rows of one cache block are contiguous, so a chunk is one or two bulk asynchronous copies each for K
//            and V (cp.async.bulk global -> shared with an mbarrier per stage); one lane requests chunk i + kStages - 1
//            before the warp starts on chunk i, so several KB per warp are in flight whatever the occupancy;
//   scores   lane = key: the lane reads its key row from shared memory 16 bytes at a time, starting at a unit rotated
//            by its lane number (rows are 128 / 256 bytes apart, so unrotated reads would all hit the same banks), and
//            forms the dot products with the G query vectors, which sit in shared memory pre-scaled;
//   softmax  per head, one max and one sum reduction per 32 keys; running (max, sum) kept per warp;
//   P V      lane = pair (D 64) or quad (D 128) of output columns: the probabilities of the chunk go through shared
//            memory, each V row is read as one conflict-free line and every lane updates its G x E accumulators.
// The warps' partial results are merged in shared memory and written in the (normalised output, max, sum) form that
// the merge kernel below combines across splits.  bf16 caches only (e4m3 stays on the kernel above); block_size must
// divide 32 or be a multiple of it.
constexpr int kPdWarps = 4;
constexpr int kPdMaxG = 8;

template <int D>
struct PdCfg {
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = 32 * kRowBytes;                       // 32 keys of K (or V)
  static constexpr int kWarpBytes = kStages * 2 * kTileBytes;             // K and V tiles of every stage
  static constexpr int kOffQ = kPdWarps * kWarpBytes;                     // float q_s[G][D]
  static constexpr int kQUnitStride = kPdMaxG * 8 + 4;                    // floats per 8-column unit of q (all heads) + pad
  static constexpr int kOffP = kOffQ + (D / 8) * kQUnitStride * 4;       // float p_s[warps][G][32]
  static constexpr int kOffBar = kOffP + kPdWarps * 32 * kPdMaxG * 4;     // mbarriers [warps][stages]
  static constexpr int kSmemBytes = kOffBar + kPdWarps * kStages * 8 + 16;
};

template <int D>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_gqa_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                        const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables,
                        const int* __restrict__ context_lens, float* __restrict__ part, int S, int Hq, int Hkv, int block_size,
                        int max_blocks, int splits, float scale, int* status) {
  using Cfg = PdCfg<D>;
  constexpr int E = D / 32;
  constexpr int ST = Cfg::kStages;
  constexpr int UNITS = D / 8;                     // 16-byte units per row
  extern __shared__ __align__(128) uint8_t pd_smem[];
  const int G = Hq / Hkv;
  const int sp = blockIdx.x % splits;
  const int hkv = (blockIdx.x / splits) % Hkv;
  const int s = blockIdx.x / (splits * Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = reinterpret_cast<float*>(pd_smem + Cfg::kOffQ);                       // [D / 8][kQUnitStride]
  float* p_s = reinterpret_cast<float*>(pd_smem + Cfg::kOffP) + warp * 32 * kPdMaxG; // [G][32] of this warp
  uint8_t* my_tiles = pd_smem + warp * Cfg::kWarpBytes;
  const uint32_t bar0 = smem_u32(pd_smem + Cfg::kOffBar) + warp * ST * 8;
  __shared__ int abort_s, drain_s;
  // the reduction at the end reuses the tile area (all copies have been consumed by then)
  // q_s[unit j][head g][8 columns], units kQUnitStride floats apart: a lane that starts at unit (lane & 7) reads 32-byte
  // pieces whose 16-byte halves fall into distinct bank groups across its quarter-warp
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    q_s[(d >> 3) * Cfg::kQUnitStride + g * 8 + (d & 7)] = __bfloat162float(q[((long long)s * Hq + hkv * G + g) * D + d]) * scale;
  }
  if (threadIdx.x == 0) { abort_s = 0; drain_s = 0; }
  if (lane == 0) {
    for (int st = 0; st < ST; ++st) mbar_init(bar0 + 8u * st, 1);
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &abort_s;
  const int ctx = context_lens[s];
  const int per = ((ctx + splits - 1) / splits + 31) / 32 * 32;      // whole 32-key chunks per split
  const int t0 = sp * per, t1 = min(ctx, t0 + per);
  const int* bt = block_tables + (long long)s * max_blocks;
  const int n_chunks = t1 > t0 ? (t1 - t0 + 31) / 32 : 0;
  const int my_n = n_chunks > warp ? (n_chunks - warp + kPdWarps - 1) / kPdWarps : 0;   // chunks warp, warp + 4, ...

  // one lane requests the K and V rows of this warp's i-th chunk into stage i % ST
  auto request = [&](int i) {
    const int c0 = t0 + (warp + i * kPdWarps) * 32;
    const uint32_t bar = bar0 + 8u * (i % ST);
    uint8_t* kt = my_tiles + (i % ST) * 2 * Cfg::kTileBytes;
    uint8_t* vt = kt + Cfg::kTileBytes;
    // rows [c0, c0 + 32) clipped to the blocks the sequence owns (the last block is allocated whole)
    const int last_row = ((t1 - 1) / block_size + 1) * block_size;            // end of the last block holding a live key
    const int r_end = min(c0 + 32, last_row);
    mbar_expect_tx(bar, uint32_t(2 * (r_end - c0) * Cfg::kRowBytes));
    for (int r = c0; r < r_end;) {
      const int blk = bt[r / block_size];
      const int in_blk = r % block_size;
      const int n = min(block_size - in_blk, r_end - r);
      const long long src = (((long long)blk * Hkv + hkv) * block_size + in_blk) * D;
      bulk_g2s_pd(smem_u32(kt + (r - c0) * Cfg::kRowBytes), k_cache + src, uint32_t(n * Cfg::kRowBytes), bar);
      bulk_g2s_pd(smem_u32(vt + (r - c0) * Cfg::kRowBytes), v_cache + src, uint32_t(n * Cfg::kRowBytes), bar);
      r += n;
    }
  };

  float m[kPdMaxG], l[kPdMaxG], acc[kPdMaxG][E];
#pragma unroll
  for (int g = 0; g < kPdMaxG; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
  }
  if (lane == 0)
    for (int i = 0; i < ST - 1 && i < my_n; ++i) request(i);
  bool ok = true;
  for (int i = 0; i < my_n; ++i) {
    if (lane == 0 && i + ST - 1 < my_n) request(i + ST - 1);      // its stage was consumed in iteration i - 1
    ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8u * (i % ST), uint32_t(i / ST) & 1u, abort_flag, status, kStatusTimeoutFull));
    if (!ok) {
      // a copy never arrived: give the other requested stages one more bounded wait each, so that no copy of this
      // warp is still writing shared memory when the CTA leaves, then drop out (the result of the CTA is discarded)
      for (int r = i + 1; r < my_n && r < i + ST; ++r)
        mbar_wait(bar0 + 8u * (r % ST), uint32_t(r / ST) & 1u, &drain_s, status, kStatusTimeoutFull);
      break;
    }
    const int c0 = t0 + (warp + i * kPdWarps) * 32;
    const uint8_t* kt = my_tiles + (i % ST) * 2 * Cfg::kTileBytes;
    const uint8_t* vt = kt + Cfg::kTileBytes;
    // ---- scores of this lane's key for every head of the group
    const bool live = c0 + lane < t1;
    float sc[kPdMaxG];
#pragma unroll
    for (int g = 0; g < kPdMaxG; ++g) sc[g] = 0.f;
    if (live) {
      const uint4* kr = reinterpret_cast<const uint4*>(kt + lane * Cfg::kRowBytes);
#pragma unroll
      for (int jj = 0; jj < UNITS; ++jj) {
        const int j = (jj + lane) & (UNITS - 1);                  // rotated start: conflict-free across the quarter-warp
        const uint4 u = kr[j];
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
#pragma unroll
        for (int g = 0; g < kPdMaxG; ++g) {
          if (g < G) {
            const float4 q0 = *reinterpret_cast<const float4*>(q_s + j * Cfg::kQUnitStride + g * 8);
            const float4 q1 = *reinterpret_cast<const float4*>(q_s + j * Cfg::kQUnitStride + g * 8 + 4);
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
        p_s[g * 32 + lane] = pv;
      }
    }
    __syncwarp();
    // ---- P V: lane = E output columns; V rows come from shared memory, one conflict-free line per key
    const int nk = min(32, t1 - c0);
#pragma unroll 4
    for (int kk = 0; kk < nk; ++kk) {
      const __nv_bfloat16* vr = reinterpret_cast<const __nv_bfloat16*>(vt + kk * Cfg::kRowBytes) + lane * E;
      float vv[E];
      if (E == 2) {
        const float2 f = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(vr));
        vv[0] = f.x; vv[1] = f.y;
      } else {
        const uint2 w2 = *reinterpret_cast<const uint2*>(vr);
        const float2 f0 = unpack_bf16x2(w2.x), f1 = unpack_bf16x2(w2.y);
        vv[0] = f0.x; vv[1] = f0.y; vv[E - 2] = f1.x; vv[E - 1] = f1.y;
      }
#pragma unroll
      for (int g = 0; g < kPdMaxG; ++g)
        if (g < G) {
          const float pgk = p_s[g * 32 + kk];              // same address for every lane: a broadcast
#pragma unroll
          for (int e = 0; e < E; ++e) acc[g][e] += pgk * vv[e];
        }
    }
    __syncwarp();            // every lane is done with this stage and with p_s before lane 0 requests into it again
  }
  // ---- merge the four warps (the tile area is free now: every requested copy has been waited for), write the partial result
  __syncthreads();
  float* red_m = reinterpret_cast<float*>(pd_smem);                 // [warps][G]
  float* red_l = red_m + kPdWarps * kPdMaxG;                         // [warps][G]
  float* red_o = red_l + kPdWarps * kPdMaxG;                         // [warps][G][D]
#pragma unroll
  for (int g = 0; g < kPdMaxG; ++g)
    if (g < G) {
      if (lane == 0) { red_m[warp * kPdMaxG + g] = ok ? m[g] : -INFINITY; red_l[warp * kPdMaxG + g] = ok ? l[g] : 0.f; }
#pragma unroll
      for (int e = 0; e < E; ++e) red_o[(warp * kPdMaxG + g) * D + lane * E + e] = acc[g][e];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i % D;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) gm = fmaxf(gm, red_m[w * kPdMaxG + g]);
    float lsum = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
      const float mw = red_m[w * kPdMaxG + g];
      if (mw == -INFINITY) continue;
      const float a = __expf(mw - gm);
      lsum += red_l[w * kPdMaxG + g] * a;
      o += red_o[(w * kPdMaxG + g) * D + d] * a;
    }
    float* out = part + (((long long)s * Hq + hkv * G + g) * splits + sp) * (D + 2);
    out[d] = lsum > 0.f ? o / lsum : 0.f;
    if (d == 0) { out[D] = gm; out[D + 1] = lsum; }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Grouped-query decode with the scores and the P V product on the warp-level tensor-core instruction.
//
// Same split of the work as paged_decode_gqa_kernel (one CTA of four warps per sequence, KV head and context split;
// a warp streams chunks of 32 keys through its own shared-memory stages), but the tiles arrive as TMA tensor copies in
// the 128-byte-swizzled layout, so that ldmatrix reads them without bank conflicts, and a chunk costs 16 ldmatrix.x4 and
// 32 mma.sync (m16n8k16: the group's query heads padded to 16 rows, 8 keys or 8 output columns per instruction) instead
// of one shared-memory pass over the whole query block per key.  The scores stay in registers: their accumulator
// fragments are, after the softmax, exactly the A fragments of the P V product.  tcgen05 is not the tool here: its
// smallest tile is 64 rows and the kernel is bound by the K / V stream, not by arithmetic.
template <int D>
struct PdMmaCfg {
  static constexpr int kStages = (D == 64) ? 3 : 2;
  static constexpr int kTileBytes = 32 * D * 2;                           // 32 keys of K (or V); D = 128: two 4 KB halves of 64 columns
  static constexpr int kWarpBytes = kStages * 2 * kTileBytes;
  static constexpr int kOffBar = kPdWarps * kWarpBytes;
  static constexpr int kSmemBytes = kOffBar + kPdWarps * kStages * 8 + 16 + 1024;   // + slack to align the tiles to 1024 bytes
};
constexpr int kPdMmaMaxG = 16;

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// tmK / tmV: the caches seen as [num_blocks * Hkv * block_size rows, D] bf16, box 64 columns x min(block_size, 32) rows,
// 128-byte swizzle.  block_size is a multiple of 8 and divides 32 or is a multiple of it.
template <int D>
__global__ void __launch_bounds__(kPdWarps * 32)
paged_decode_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_tables,
                        const int* __restrict__ context_lens, float* __restrict__ part, int S, int Hq, int Hkv, int block_size,
                        int max_blocks, int splits, float scale, int* status) {
  using Cfg = PdMmaCfg<D>;
  constexpr int ST = Cfg::kStages;
  constexpr int KS = D / 16;     // k-steps of the score product
  constexpr int NT = D / 8;      // 8-column blocks of the output
  extern __shared__ uint8_t pd_raw[];
  uint8_t* pd_smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pd_raw) + 1023) & ~uintptr_t(1023));
  const int G = Hq / Hkv;
  const int sp = blockIdx.x % splits;
  const int hkv = (blockIdx.x / splits) % Hkv;
  const int s = blockIdx.x / (splits * Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, qd = lane & 3;
  uint8_t* my_tiles = pd_smem + warp * Cfg::kWarpBytes;
  const uint32_t bar0 = smem_u32(pd_smem + Cfg::kOffBar) + warp * ST * 8;
  __shared__ int abort_s, drain_s;
  if (threadIdx.x == 0) { abort_s = 0; drain_s = 0; }
  if (lane == 0) {
    for (int st = 0; st < ST; ++st) mbar_init(bar0 + 8u * st, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  // A fragments of the query block: rows = heads of the group (g and g + 8), zero past G
  uint32_t qa[KS][4];
  {
    const bool lo = g < G, hi = g + 8 < G;
    const __nv_bfloat16* qlo = q + ((long long)s * Hq + hkv * G + (lo ? g : 0)) * D + qd * 2;
    const __nv_bfloat16* qhi = q + ((long long)s * Hq + hkv * G + (hi ? g + 8 : 0)) * D + qd * 2;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      qa[kk][0] = lo ? *reinterpret_cast<const uint32_t*>(qlo + kk * 16) : 0u;
      qa[kk][1] = hi ? *reinterpret_cast<const uint32_t*>(qhi + kk * 16) : 0u;
      qa[kk][2] = lo ? *reinterpret_cast<const uint32_t*>(qlo + kk * 16 + 8) : 0u;
      qa[kk][3] = hi ? *reinterpret_cast<const uint32_t*>(qhi + kk * 16 + 8) : 0u;
    }
  }
  __syncthreads();
  volatile int* abort_flag = &abort_s;
  const int ctx = context_lens[s];
  const int per = ((ctx + splits - 1) / splits + 31) / 32 * 32;      // whole 32-key chunks per split
  const int t0 = sp * per, t1 = min(ctx, t0 + per);
  const int* bt = block_tables + (long long)s * max_blocks;
  const int n_chunks = t1 > t0 ? (t1 - t0 + 31) / 32 : 0;
  const int my_n = n_chunks > warp ? (n_chunks - warp + kPdWarps - 1) / kPdWarps : 0;   // chunks warp, warp + 4, ...
  const int run = block_size < 32 ? block_size : 32;                 // rows per tensor copy

  auto request = [&](int i) {
    const int c0 = t0 + (warp + i * kPdWarps) * 32;
    const uint32_t bar = bar0 + 8u * (i % ST);
    uint8_t* kt = my_tiles + (i % ST) * 2 * Cfg::kTileBytes;
    uint8_t* vt = kt + Cfg::kTileBytes;
    const int last_row = ((t1 - 1) / block_size + 1) * block_size;   // end of the last block holding a live key
    const int r_end = min(c0 + 32, last_row);
    mbar_expect_tx(bar, uint32_t(2 * (r_end - c0) * D * 2));
    for (int r = c0; r < r_end; r += run) {
      const int blk = bt[r / block_size];
      const int row = (blk * Hkv + hkv) * block_size + r % block_size;
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        tma_load_2d(smem_u32(kt + h * 4096 + (r - c0) * 128), &tmK, bar, h * 64, row);
        tma_load_2d(smem_u32(vt + h * 4096 + (r - c0) * 128), &tmV, bar, h * 64, row);
      }
    }
  };

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;   // l: this lane's share of the row sums
  float oacc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int r = 0; r < 4; ++r) oacc[nt][r] = 0.f;

  if (lane == 0)
    for (int i = 0; i < ST - 1 && i < my_n; ++i) request(i);
  bool ok = true;
  const int lj = lane >> 3, lr = lane & 7;   // ldmatrix: this lane addresses row lr of matrix lj
  for (int i = 0; i < my_n; ++i) {
    if (lane == 0 && i + ST - 1 < my_n) request(i + ST - 1);      // its stage was consumed in iteration i - 1
    ok = __all_sync(0xffffffffu, mbar_wait(bar0 + 8u * (i % ST), uint32_t(i / ST) & 1u, abort_flag, status, kStatusTimeoutFull));
    if (!ok) {
      // a copy never arrived: give the other requested stages one more bounded wait each, so that no copy of this
      // warp is still writing shared memory when the CTA leaves, then drop out (the result of the CTA is discarded)
      for (int r = i + 1; r < my_n && r < i + ST; ++r)
        mbar_wait(bar0 + 8u * (r % ST), uint32_t(r / ST) & 1u, &drain_s, status, kStatusTimeoutFull);
      break;
    }
    const int c0 = t0 + (warp + i * kPdWarps) * 32;
    uint8_t* kt = my_tiles + (i % ST) * 2 * Cfg::kTileBytes;
    uint8_t* vt = kt + Cfg::kTileBytes;
    const uint32_t kt_addr = smem_u32(kt), vt_addr = smem_u32(vt);
    const int nk = min(32, t1 - c0);
    if (nk < 32) {
      // rows past the context (the tail of the last block, or never copied) may hold anything: zero them in V so that
      // their zero probabilities do not meet a NaN
      if (lane >= nk) {
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          uint4* row = reinterpret_cast<uint4*>(vt + h * 4096 + lane * 128);
#pragma unroll
          for (int u = 0; u < 8; ++u) row[u] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      __syncwarp();
    }
    // ---- S = Q K^T: four blocks of 8 keys
    float sacc[4][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
      for (int r = 0; r < 4; ++r) sacc[t][r] = 0.f;
      const int key = t * 8 + lr;
#pragma unroll
      for (int kk2 = 0; kk2 < KS / 2; ++kk2) {
        const int u = kk2 * 4 + lj;                                 // 16-byte unit of the row: columns 8 u .. 8 u + 7
        uint32_t b00, b01, b10, b11;
        ldsm_x4(kt_addr + (u >> 3) * 4096 + key * 128 + (((u & 7) ^ (key & 7)) << 4), b00, b01, b10, b11);
        mma_16816(sacc[t], qa[2 * kk2], b00, b01);
        mma_16816(sacc[t], qa[2 * kk2 + 1], b10, b11);
      }
    }
    // ---- online softmax: this lane holds columns t * 8 + qd * 2 + {0, 1} of rows g (registers 0, 1) and g + 8 (2, 3)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool live = t * 8 + qd * 2 + e < nk;
        sacc[t][e] = live ? sacc[t][e] * scale : -INFINITY;
        sacc[t][2 + e] = live ? sacc[t][2 + e] * scale : -INFINITY;
        mx_lo = fmaxf(mx_lo, sacc[t][e]);
        mx_hi = fmaxf(mx_hi, sacc[t][2 + e]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float nm_lo = fmaxf(m_lo, mx_lo), nm_hi = fmaxf(m_hi, mx_hi);   // finite: every chunk has a live key
    const float a_lo = (m_lo == -INFINITY) ? 0.f : __expf(m_lo - nm_lo);
    const float a_hi = (m_hi == -INFINITY) ? 0.f : __expf(m_hi - nm_hi);
    m_lo = nm_lo; m_hi = nm_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
    uint32_t pa[2][4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float p0 = __expf(sacc[t][0] - nm_lo), p1 = __expf(sacc[t][1] - nm_lo);
      const float p2 = __expf(sacc[t][2] - nm_hi), p3 = __expf(sacc[t][3] - nm_hi);
      ps_lo += p0 + p1;
      ps_hi += p2 + p3;
      pa[t >> 1][(t & 1) * 2] = pack_bf16x2(p0, p1);         // keys 16 ks + 8 (t & 1) + ..: registers 0 / 2 rows g, 1 / 3 rows g + 8
      pa[t >> 1][(t & 1) * 2 + 1] = pack_bf16x2(p2, p3);
    }
    l_lo = l_lo * a_lo + ps_lo;
    l_hi = l_hi * a_hi + ps_hi;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      oacc[nt][0] *= a_lo; oacc[nt][1] *= a_lo;
      oacc[nt][2] *= a_hi; oacc[nt][3] *= a_hi;
    }
    // ---- O += P V: two steps of 16 keys, transposed loads of V
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const int key = ks * 16 + (lj & 1) * 8 + lr;
#pragma unroll
      for (int nt2 = 0; nt2 < NT / 2; ++nt2) {
        const int u = nt2 * 2 + (lj >> 1);
        uint32_t b0a, b1a, b0b, b1b;
        ldsm_x4_trans(vt_addr + (u >> 3) * 4096 + key * 128 + (((u & 7) ^ (key & 7)) << 4), b0a, b1a, b0b, b1b);
        mma_16816(oacc[2 * nt2], pa[ks], b0a, b1a);
        mma_16816(oacc[2 * nt2 + 1], pa[ks], b0b, b1b);
      }
    }
    __syncwarp();            // every lane is done with this stage before lane 0 requests into it again
  }
  // ---- merge the four warps (the tile area is free now: every requested copy has been waited for), write the partial result
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  __syncthreads();
  float* red_m = reinterpret_cast<float*>(pd_smem);                 // [warps][16]
  float* red_l = red_m + kPdWarps * kPdMmaMaxG;                      // [warps][16]
  float* red_o = red_l + kPdWarps * kPdMmaMaxG;                      // [warps][16][D]
  if (qd == 0) {
    red_m[warp * kPdMmaMaxG + g] = ok ? m_lo : -INFINITY;
    red_l[warp * kPdMmaMaxG + g] = ok ? l_lo : 0.f;
    red_m[warp * kPdMmaMaxG + g + 8] = ok ? m_hi : -INFINITY;
    red_l[warp * kPdMmaMaxG + g + 8] = ok ? l_hi : 0.f;
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float* lo = red_o + (warp * kPdMmaMaxG + g) * D + nt * 8 + qd * 2;
    float* hi = red_o + (warp * kPdMmaMaxG + g + 8) * D + nt * 8 + qd * 2;
    *reinterpret_cast<float2*>(lo) = make_float2(oacc[nt][0], oacc[nt][1]);
    *reinterpret_cast<float2*>(hi) = make_float2(oacc[nt][2], oacc[nt][3]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int gg = i / D, d = i % D;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) gm = fmaxf(gm, red_m[w * kPdMmaMaxG + gg]);
    float lsum = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kPdWarps; ++w) {
      const float mw = red_m[w * kPdMmaMaxG + gg];
      if (mw == -INFINITY) continue;
      const float a = __expf(mw - gm);
      lsum += red_l[w * kPdMmaMaxG + gg] * a;
      o += red_o[(w * kPdMmaMaxG + gg) * D + d] * a;
    }
    float* out = part + (((long long)s * Hq + hkv * G + gg) * splits + sp) * (D + 2);
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
// part: scratch [S, Hq, splits, D + 2] fp32; o: [S, Hq, D] bf16.  num_blocks: blocks in the caches (0: not known, which
// rules out the tensor-copy kernel).
int lt_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables, const int* context_lens,
                    float* part, void* o, int S, int Hq, int Hkv, int D, int block_size, int max_blocks, int num_blocks,
                    int splits, float scale, int kv_fp8, float k_scale, float v_scale, void* stream) {
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
  const bool bs_ok = block_size > 0 && (32 % block_size == 0 || block_size % 32 == 0);
  const bool aligned = (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0;
  if (!kv_fp8 && G <= kPdMmaMaxG && bs_ok && block_size % 8 == 0 && num_blocks > 0 && aligned &&
      (long long)num_blocks * Hkv * block_size < (1ll << 31)) {
    // bf16 caches in blocks of 8 keys or more: tiles by TMA in the swizzled layout, scores and P V on mma.sync
    const int ctas = S * Hkv * splits;
    static bool configured_mma = false;
    if (!configured_mma) {
      LT_RETURN_IF_CUDA(cudaFuncSetAttribute(paged_decode_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PdMmaCfg<64>::kSmemBytes));
      LT_RETURN_IF_CUDA(cudaFuncSetAttribute(paged_decode_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PdMmaCfg<128>::kSmemBytes));
      configured_mma = true;
    }
    const uint64_t rows = uint64_t(num_blocks) * Hkv * block_size;
    const uint32_t run = block_size < 32 ? block_size : 32;
    CUtensorMap tmK, tmV;
    int r = encode_tmap_2d(&tmK, k_cache, 2, D, rows, uint64_t(D) * 2, 64, run, 1);
    if (r == 0) r = encode_tmap_2d(&tmV, v_cache, 2, D, rows, uint64_t(D) * 2, 64, run, 1);
    if (r) return r > 0 ? 1000 + r : r;
    int* status = device_status_word();
    if (D == 64) paged_decode_mma_kernel<64><<<ctas, kPdWarps * 32, PdMmaCfg<64>::kSmemBytes, st>>>(tmK, tmV, Q, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale, status);
    else paged_decode_mma_kernel<128><<<ctas, kPdWarps * 32, PdMmaCfg<128>::kSmemBytes, st>>>(tmK, tmV, Q, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale, status);
  } else if (!kv_fp8 && G <= kPdMaxG && bs_ok && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_cache) & 15) == 0) {
    // bf16 caches: every K / V byte is read once for the whole group of query heads, through a shared-memory pipeline
    const int ctas = S * Hkv * splits;
    auto KC = static_cast<const __nv_bfloat16*>(k_cache);
    auto VC = static_cast<const __nv_bfloat16*>(v_cache);
    static bool configured = false;
    if (!configured) {
      LT_RETURN_IF_CUDA(cudaFuncSetAttribute(paged_decode_gqa_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PdCfg<64>::kSmemBytes));
      LT_RETURN_IF_CUDA(cudaFuncSetAttribute(paged_decode_gqa_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PdCfg<128>::kSmemBytes));
      configured = true;
    }
    int* status = device_status_word();
    if (D == 64) paged_decode_gqa_kernel<64><<<ctas, kPdWarps * 32, PdCfg<64>::kSmemBytes, st>>>(Q, KC, VC, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale, status);
    else paged_decode_gqa_kernel<128><<<ctas, kPdWarps * 32, PdCfg<128>::kSmemBytes, st>>>(Q, KC, VC, block_tables, context_lens, part, S, Hq, Hkv, block_size, max_blocks, splits, scale, status);
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
