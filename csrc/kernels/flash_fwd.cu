// FlashAttention forward for sm_100a: causal or full, grouped-query heads, bf16, head_dim 64 or 128.
//
// The reference's CUDA attention materialises S = Q K^T for all heads in fp32 (four B*H*Tq*Tk scratch
// buffers), runs a row-softmax kernel and a second batched GEMM, has no causal mask and ignores the number
// of KV heads (src/backend/gpu_native/nn/flash_attention.cu:188-299).  This kernel never leaves the chip:
//
//   warp 0    TMA producer: Q tile once, K/V tiles double-buffered (128-byte swizzle, mbarrier tx)
//   warp 1    MMA issuer:   S_j = Q K_j^T  (tcgen05.mma, 128x128xD, S double-buffered in TMEM)
//                           O  += P_j V_j  (A = P_j from shared memory, B = V_j as an N-major operand)
//   warps 2-5 softmax:      one query row per thread (TMEM lane = row): tcgen05.ld S, online max / sum in
//                           the exp2 domain, P_j written to shared memory in the swizzled operand layout.
// The running maximum is updated lazily: O in TMEM is rescaled only when a row's maximum grew by more
// than 2^8, which keeps exp2 arguments bounded and makes the rescale (tcgen05.ld/st of O) rare.
// Output: O [B, Tq, Hq, D] bf16 and the natural-log LSE [B, Hq, Tq] fp32 for the backward pass.
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kFaBlockQ = 128;
constexpr int kFaBlockKV = 128;
constexpr int kFaThreads = 352;          // warp 0 producer, warp 1 PV MMA issuer, warps 2-9 softmax, warp 10 score MMA issuer
constexpr int kFaSoftmaxThreads = 256;   // two warps per TMEM lane quarter, 64 score columns each

struct FlashFwdParams {
  __nv_bfloat16* O;
  float* lse;
  int B, Tq, Tk, Hq, Hkv;
  long long so_b, so_t;
  float scale_log2;  // softmax scale * log2(e)
  int causal;
  int* status;
  long long* trace;   // optional phase timing of one CTA (debug aid; nullptr = off), 16 int64
  // Context parallelism: the keys/values of cp_world ranks (Tk rows each, read through per-rank tensor maps that may
  // point at peer memory) are visited in one pass; queries and keys carry global positions (contiguous split, or
  // zigzag: rank r holds sequence chunks r and 2W-1-r of 2W).  cp_world == 1 is plain attention.
  int cp_world, cp_rank, zigzag;
};

constexpr int kFaMaxRanks = 8;
struct KvMaps {
  CUtensorMap k[kFaMaxRanks];
  CUtensorMap v[kFaMaxRanks];
};

// A run of consecutive visible KV blocks of one rank.
struct KvSeg {
  int n, owner, kv0, kbase;
};
constexpr int kFaMaxSegs = 2 * kFaMaxRanks;

__device__ __forceinline__ float ex2_approx_f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct FaFwdCfg {
  static constexpr int kQBytes = kFaBlockQ * D * 2;
  static constexpr int kKVBytes = kFaBlockKV * D * 2;
  static constexpr int kPBytes = kFaBlockQ * kFaBlockKV * 2;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kQBytes;
  static constexpr int kOffV = kOffK + 2 * kKVBytes;
  static constexpr int kOffP = kOffV + 2 * kKVBytes;
  static constexpr int kOffBar = kOffP + 2 * kPBytes;
  static constexpr int kOffSeg = kOffBar + 224;               // KvSeg table (16 entries) + block count
  static constexpr int kOffX = kOffSeg + kFaMaxSegs * 16 + 16;                 // row statistics exchanged between the two column halves
  static constexpr int kNeeded = kOffX + 2 * 2 * 128 * 4;     // [parity][half][128] floats
  // 1 KB of slack for the 1024-byte alignment where it fits under the 227 KB limit; the kernel checks at run time
  // that the aligned layout lies inside the allocation and reports kStatusBadArgument otherwise.
  static constexpr int kSmemBytes = (kNeeded + 1024 <= 232448) ? kNeeded + 1024 : 232448;
  static constexpr int kTmemCols = 512;
  // Score buffers of 128 columns: three with head_dim 64, so that S of block j+2 is computed while the softmax of
  // blocks j and j+1 is still reading theirs; tensor memory only has room for two with head_dim 128.
  static constexpr int kSBufs = (D == 64) ? 3 : 2;
  static constexpr int kColS = 0;
  static constexpr int kColO = kSBufs * 128;   // two accumulators of D columns (KV blocks of even / odd index)
};

template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ KvMaps maps, const FlashFwdParams p) {
  using Cfg = FaFwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  if (int(smem - smem_raw) + Cfg::kNeeded > Cfg::kSmemBytes) {  // uniform for the whole grid
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, int(kStatusBadArgument));
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  const uint32_t bb = smem_u32(bars);
  // barrier map
  const uint32_t q_full = bb;
  auto k_full = [&](int s) { return bb + 8u * (1 + s); };
  auto v_full = [&](int s) { return bb + 8u * (3 + s); };
  auto k_empty = [&](int s) { return bb + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bb + 8u * (7 + s); };
  auto s_full = [&](int s) { return bb + 8u * (9 + s); };    // up to three
  auto p_full = [&](int s) { return bb + 8u * (12 + s); };
  auto p_empty = [&](int s) { return bb + 8u * (14 + s); };
  const uint32_t o_full = bb + 8u * 16;
  // x_bar(quarter): both warps of a TMEM lane quarter have published their partial row statistics
  auto x_bar = [&](int qtr) { return bb + 8u * (17 + qtr); };
  auto s_free = [&](int sb) { return bb + 8u * (21 + sb); };   // the group's four warps have read score buffer sb
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 24);
  float* xmax = reinterpret_cast<float*>(smem + Cfg::kOffX);  // [2 (rendezvous parity)][2 (half)][128]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Launch order is x fastest: every head and batch entry of the heaviest (latest) query block runs before any
  // lighter block, and neighbouring CTAs are the query heads that share one KV head (the K/V tiles stay in L2).
  const int q_blk = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / (p.Hq / p.Hkv);
  const int q0 = q_blk * kFaBlockQ;
  KvSeg* segs = reinterpret_cast<KvSeg*>(smem + Cfg::kOffSeg);
  int* n_blocks_s = reinterpret_cast<int*>(smem + Cfg::kOffSeg + kFaMaxSegs * 16);
  // global position of this block's first query
  int q_base;
  if (p.cp_world == 1) {
    q_base = q0 + (p.Tk - p.Tq);  // key index visible to query i is <= i + (Tk - Tq)
  } else if (p.zigzag) {
    const int hq = p.Tq / 2;
    q_base = q0 < hq ? p.cp_rank * hq + q0 : (2 * p.cp_world - 1 - p.cp_rank) * hq + (q0 - hq);
  } else {
    q_base = p.cp_rank * p.Tq + q0;
  }
  if (threadIdx.x == 0) {
    // visible KV blocks as runs: own rank first (local memory), then the other ranks
    const int q_last = q_base + kFaBlockQ - 1;
    const int nb_all = (p.Tk + kFaBlockKV - 1) / kFaBlockKV;
    int ns = 0, total = 0;
    for (int i = 0; i < p.cp_world; ++i) {
      const int o = (p.cp_rank + i) % p.cp_world;
      const int parts = (p.cp_world > 1 && p.zigzag) ? 2 : 1;
      for (int h2 = 0; h2 < parts; ++h2) {
        int kv0, kbase, nb;
        if (parts == 2) {
          const int hk = p.Tk / 2;
          kv0 = h2 * hk;
          kbase = h2 == 0 ? o * hk : (2 * p.cp_world - 1 - o) * hk;
          nb = hk / kFaBlockKV;
        } else {
          kv0 = 0;
          kbase = p.cp_world > 1 ? o * p.Tk : 0;
          nb = nb_all;
        }
        if (p.causal) {
          const int vis = q_last < kbase ? 0 : (q_last - kbase) / kFaBlockKV + 1;
          nb = nb < vis ? nb : vis;
        }
        if (nb > 0) {
          segs[ns] = KvSeg{nb, o, kv0, kbase};
          ++ns;
          total += nb;
        }
      }
    }
    for (int i = ns; i < kFaMaxSegs; ++i) segs[i] = KvSeg{0, 0, 0, 0};
    *n_blocks_s = total;
  }
  __syncthreads();
  const int n_blocks = *n_blocks_s;
  // block j of the schedule -> (owner rank, first local key row, global position of its first key)
  auto locate = [&](int j, int& owner, int& kv0, int& kbase) {
    int sidx = 0;
    while (sidx < kFaMaxSegs - 1 && j >= segs[sidx].n) { j -= segs[sidx].n; ++sidx; }
    owner = segs[sidx].owner;
    kv0 = segs[sidx].kv0 + j * kFaBlockKV;
    kbase = segs[sidx].kbase + j * kFaBlockKV;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1); mbar_init(v_full(s), 1);
      mbar_init(k_empty(s), 1); mbar_init(v_empty(s), 1);
      mbar_init(p_full(s), kFaSoftmaxThreads / 64); mbar_init(p_empty(s), 1);
    }
    for (int s = 0; s < Cfg::kSBufs; ++s) { mbar_init(s_full(s), 1); mbar_init(s_free(s), kFaSoftmaxThreads / 64); }
    mbar_init(o_full, 1);
    for (int qtr = 0; qtr < 4; ++qtr) mbar_init(x_bar(qtr), 2);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&maps.k[p.cp_rank]); tma_prefetch_desc(&maps.v[p.cp_rank]);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && n_blocks > 0) {
      mbar_expect_tx(q_full, Cfg::kQBytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_load_4d(sbase + Cfg::kOffQ + c * (kFaBlockQ * 128), &tmQ, q_full, c * 64, h, q0, b);
      // K runs one block ahead of V: the wait for a free V stage (the PV product two blocks back) must not hold up
      // the K tile that the next score product needs.
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        int owner, kv0, kbase;
        locate(j, owner, kv0, kbase);
        if (!mbar_wait(k_empty(s), ((j >> 1) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) return false;
        mbar_expect_tx(k_full(s), Cfg::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(sbase + Cfg::kOffK + s * Cfg::kKVBytes + c * (kFaBlockKV * 128), &maps.k[owner], k_full(s), c * 64, hkv,
                      kv0, b);
        return true;
      };
      bool okp = load_k(0);
      for (int j = 0; okp && j < n_blocks; ++j) {
        if (j + 1 < n_blocks && !load_k(j + 1)) break;
        const int s = j & 1;
        int owner, kv0, kbase;
        locate(j, owner, kv0, kbase);
        if (!mbar_wait(v_empty(s), ((j >> 1) & 1) ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        mbar_expect_tx(v_full(s), Cfg::kKVBytes);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_4d(sbase + Cfg::kOffV + s * Cfg::kKVBytes + c * (kFaBlockKV * 128), &maps.v[owner], v_full(s), c * 64, hkv,
                      kv0, b);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- score MMA issuer (S = Q K^T)
    // Issuing a tcgen05.mma costs its thread on the order of a hundred cycles whatever the tile width, so the twelve
    // MMAs of a KV block are split over two issuing threads: this one runs the score products as far ahead as the
    // score buffers allow, warp 1 runs the PV products.
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kFaBlockQ, kFaBlockKV, 1, 0, 0);
      const uint64_t q_desc = make_smem_desc_sw128(sbase + Cfg::kOffQ, 16, 1024);
      const uint64_t k_desc0 = make_smem_desc_sw128(sbase + Cfg::kOffK, 16, 1024);
      const uint64_t k_desc1 = make_smem_desc_sw128(sbase + Cfg::kOffK + Cfg::kKVBytes, 16, 1024);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusTimeoutFull);
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int s = j & 1;                 // K stage
        const int sb = j % Cfg::kSBufs;      // score buffer, last read by the softmax of block j - kSBufs
        if (!mbar_wait(k_full(s), (j >> 1) & 1, abort_flag, p.status, kStatusTimeoutFull)) break;
        if (j >= Cfg::kSBufs &&
            !mbar_wait(s_free(sb), uint32_t(j / Cfg::kSBufs - 1) & 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint64_t kd = s ? k_desc1 : k_desc0;
        const uint32_t d_s = tmem_base + Cfg::kColS + sb * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t off = uint64_t(((k / 4) * (128 * 128) + (k % 4) * 32) >> 4);   // 16-byte units
          umma_f16_ss(d_s, q_desc + off, kd + off, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(k_empty(s));
        umma_commit(s_full(sb));
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- PV MMA issuer (O_g += P V)
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_o = make_idesc_f16(kFaBlockQ, D, 1, 0, 1);
      uint64_t v_desc[2], p_desc[2];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        v_desc[st] = make_smem_desc_sw128(sbase + Cfg::kOffV + st * Cfg::kKVBytes, kFaBlockKV * 128, 1024);
        p_desc[st] = make_smem_desc_sw128(sbase + Cfg::kOffP + st * Cfg::kPBytes, 16, 1024);
      }
      const bool trm = p.trace != nullptr && blockIdx.z == 0 && h == 0 && b == 0;
      long long tm[3] = {0, 0, 0};
      bool ok = true;
      for (int j = 0; ok && j < n_blocks; ++j) {
        const int s = j & 1;
        const uint32_t par = (j >> 1) & 1;
        long long c0 = trm ? clock64() : 0;
        if (!mbar_wait(p_full(s), par, abort_flag, p.status, kStatusTimeoutTmemFull)) { ok = false; break; }
        if (trm) { const long long c1 = clock64(); tm[1] += c1 - c0; c0 = c1; }   // waiting for P
        if (!mbar_wait(v_full(s), par, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
        if (trm) { const long long c1 = clock64(); tm[2] += c1 - c0; c0 = c1; }   // waiting for V
        tc_fence_after();
        const uint64_t pd = s ? p_desc[1] : p_desc[0];
        const uint64_t vd = s ? v_desc[1] : v_desc[0];
        const uint32_t d_o = tmem_base + Cfg::kColO + s * D;
#pragma unroll
        for (int k = 0; k < kFaBlockKV / 16; ++k) {
          const uint64_t a_off = uint64_t(((k / 4) * (128 * 128) + (k % 4) * 32) >> 4);
          const uint64_t b_off = uint64_t((k * (16 * 128)) >> 4);
          umma_f16_ss(d_o, pd + a_off, vd + b_off, idesc_o, (j > 1 || k > 0) ? 1u : 0u);
        }
        umma_commit(v_empty(s));
        umma_commit(p_empty(s));
        if (j == n_blocks - 1) umma_commit(o_full);
        if (trm) { const long long c1 = clock64(); tm[0] += c1 - c0; c0 = c1; }   // issuing the PV MMAs
      }
      if (trm) { p.trace[8] = tm[0]; p.trace[9] = tm[1]; p.trace[10] = tm[2]; p.trace[11] = n_blocks; }
    }
  } else if (warp < 10) {
    // ---------------------------------------------------------------- softmax + epilogue
    // Two independent groups of four warps: group g takes the KV blocks of parity g (score buffer g, P buffer g) and
    // keeps its own running maximum, row sum and output accumulator O_g, so a thread owns a whole score row of its
    // block (no exchange of row statistics between warps) and the softmax of block j+1 overlaps that of block j.
    // The two accumulators are merged once, at the end.
    const int quarter = warp & 3;          // TMEM lanes this warp may touch
    const int grp = (warp - 2) >> 2;       // which blocks (and, in the epilogue, which half of the output columns)
    const int row = quarter * 32 + lane;
    const int q_idx = q0 + row;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t o_mine = tmem_base + lane_base + Cfg::kColO + grp * D;
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    const bool tr = p.trace != nullptr && blockIdx.z == 0 && h == 0 && b == 0 && warp == 2 && lane == 0;
    long long tc[6] = {0, 0, 0, 0, 0, 0};
    int tn = 0;
    for (int j = grp; j < n_blocks; j += 2) {
      long long c0 = tr ? clock64() : 0;
      ++tn;
      const uint32_t par = (j >> 1) & 1;
      const int sb = j % Cfg::kSBufs;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full(sb), uint32_t(j / Cfg::kSBufs) & 1u, abort_flag, p.status,
                                             kStatusTimeoutTmemFull));
      if (!ok) break;
      if (tr) { const long long c1 = clock64(); tc[0] += c1 - c0; c0 = c1; }   // waiting for S
      tc_fence_after();
      int owner, kv0b, kbase;
      locate(j, owner, kv0b, kbase);
      // last visible column of this 128-key block for this row: causal position and end of the rank's keys
      int limit = p.Tk - 1 - kv0b;
      if (p.causal) limit = min(limit, q_base + row - kbase);
      const uint32_t s_mine = tmem_base + lane_base + Cfg::kColS + sb * 128;
      // pass 1: row maximum (the scores are read from tensor memory twice, 64 columns at a time, instead of
      // holding all 128 in registers)
      float mx = -INFINITY;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t r[2][32];
        tmem_ld_32x32(s_mine + hh * 64, r[0]);
        tmem_ld_32x32(s_mine + hh * 64 + 32, r[1]);
        tmem_ld_wait();
        if (limit >= hh * 64 + 63) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[c][i]));
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (hh * 64 + c * 32 + i <= limit) mx = fmaxf(mx, __uint_as_float(r[c][i]));
        }
      }
      if (tr) { const long long c1 = clock64(); tc[1] += c1 - c0; c0 = c1; }   // pass 1 (row maximum)
      const float m_blk = mx * p.scale_log2;
      if (j == grp) {
        m_used = (m_blk == -INFINITY) ? 0.f : m_blk;
      } else {
        const float m_new = fmaxf(m_used, m_blk);
        const bool need = (m_new - m_used > 8.f);
        if (__any_sync(0xffffffffu, need)) {
          // O_g must be complete up to this group's previous block before it is rescaled.
          ok = __all_sync(0xffffffffu, mbar_wait(p_empty(grp), par ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty));
          if (!ok) break;
          tc_fence_after();
          const float alpha = need ? ex2_approx_f(m_used - m_new) : 1.f;
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(o_mine + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(o_mine + c * 16, o);
          }
          tmem_st_wait();
          l *= alpha;
          if (need) m_used = m_new;
        }
      }
      if (tr) { const long long c1 = clock64(); tc[2] += c1 - c0; c0 = c1; }   // rescale of O (rare)
      // P buffer g is free once this group's previous PV has been executed.
      ok = __all_sync(0xffffffffu, mbar_wait(p_empty(grp), par ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty));
      if (!ok) break;
      if (tr) { const long long c1 = clock64(); tc[3] += c1 - c0; c0 = c1; }   // waiting for the P buffer
      // pass 2: exponentials, row sum, bf16 P into the swizzled operand tile (64 keys = one 128-byte row chunk)
      float sum = 0.f;
      uint8_t* prow = smem + Cfg::kOffP + grp * Cfg::kPBytes + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t r[2][32];
        tmem_ld_32x32(s_mine + hh * 64, r[0]);
        tmem_ld_32x32(s_mine + hh * 64 + 32, r[1]);
        tmem_ld_wait();
        const bool full_vis = (limit >= hh * 64 + 63);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float pv = ex2_approx_f(fmaf(__uint_as_float(r[c][i]), p.scale_log2, -m_used));
            if (!full_vis && hh * 64 + c * 32 + i > limit) pv = 0.f;
            sum += pv;
            r[c][i] = __float_as_uint(pv);
          }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(r[c][u * 8 + 0]), __uint_as_float(r[c][u * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(r[c][u * 8 + 2]), __uint_as_float(r[c][u * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(r[c][u * 8 + 4]), __uint_as_float(r[c][u * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(r[c][u * 8 + 6]), __uint_as_float(r[c][u * 8 + 7]));
            const int unit = (c * 4 + u) ^ (row & 7);  // 16-byte unit inside the 128-byte row of key chunk hh
            *reinterpret_cast<uint4*>(prow + hh * (128 * 128) + unit * 16) = w;
          }
        }
      }
      l += sum;
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {   // one arrival per warp of the group
        mbar_arrive(s_free(sb));
        mbar_arrive(p_full(grp));
      }
      if (tr) { const long long c1 = clock64(); tc[4] += c1 - c0; c0 = c1; }   // pass 2 (exp, P stores, fence, arrive)
    }
    if (tr) {
      for (int i = 0; i < 5; ++i) p.trace[i] = tc[i];
      p.trace[15] = tn;
    }
    if (ok && n_blocks > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(o_full, 0, abort_flag, p.status, kStatusTimeoutTmemFull));
    }
    // merge the two groups: exchange (maximum, row sum) with the warp of the other group on the same lane quarter
    const bool mine_used = n_blocks > grp, other_used = n_blocks > (grp ^ 1);
    float m_o = 0.f, l_o = 0.f;
    if (ok) {
      xmax[(grp * 2 + 0) * 128 + row] = m_used;
      xmax[(grp * 2 + 1) * 128 + row] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar(quarter));
      ok = __all_sync(0xffffffffu, mbar_wait(x_bar(quarter), 0, abort_flag, p.status, kStatusTimeoutLocalFlag));
      if (ok) {
        m_o = xmax[((grp ^ 1) * 2 + 0) * 128 + row];
        l_o = xmax[((grp ^ 1) * 2 + 1) * 128 + row];
      }
    }
    if (ok) {
      float m_all = m_used, a_mine = 1.f, a_other = 0.f;
      if (mine_used && other_used) {
        m_all = fmaxf(m_used, m_o);
        a_mine = ex2_approx_f(m_used - m_all);
        a_other = ex2_approx_f(m_o - m_all);
      } else if (!mine_used && other_used) {
        m_all = m_o; a_mine = 0.f; a_other = 1.f;
      }
      const float l_all = (mine_used ? l * a_mine : 0.f) + (other_used ? l_o * a_other : 0.f);
      const float inv_l = (l_all > 0.f) ? 1.f / l_all : 0.f;
      const float w_mine = a_mine * inv_l, w_other = a_other * inv_l;
      if (n_blocks > 0) tc_fence_after();
      __nv_bfloat16* orow = p.O + (long long)b * p.so_b + (long long)q_idx * p.so_t + (long long)h * D;
      const uint32_t o_other = tmem_base + lane_base + Cfg::kColO + (grp ^ 1) * D;
      // this warp writes output columns [grp * D / 2, (grp + 1) * D / 2) of its 32 rows
#pragma unroll 1
      for (int c = grp * (D / 32); c < (grp + 1) * (D / 32); ++c) {
        uint32_t o[16], o2[16];
        if (mine_used) tmem_ld_32x16(o_mine + c * 16, o);
        if (other_used) tmem_ld_32x16(o_other + c * 16, o2);
        if (mine_used || other_used) tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float acc = 0.f;
          if (mine_used) acc = __uint_as_float(o[i]) * w_mine;
          if (other_used) acc = fmaf(__uint_as_float(o2[i]), w_other, acc);
          v[i] = acc;
        }
        if (q_idx < p.Tq) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            uint4 w;
            w.x = pack_bf16x2(v[u * 8 + 0], v[u * 8 + 1]);
            w.y = pack_bf16x2(v[u * 8 + 2], v[u * 8 + 3]);
            w.z = pack_bf16x2(v[u * 8 + 4], v[u * 8 + 5]);
            w.w = pack_bf16x2(v[u * 8 + 6], v[u * 8 + 7]);
            *reinterpret_cast<uint4*>(orow + c * 16 + u * 8) = w;
          }
        }
      }
      if (grp == 0 && q_idx < p.Tq)
        p.lse[((long long)b * p.Hq + h) * p.Tq + q_idx] = (l_all > 0.f) ? (m_all + log2f(l_all)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int spin = 0; spin < 2000; ++spin) __nanosleep(100);  // bounded grace period for copies in flight
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

static long long* g_fwd_trace = nullptr;

template <int D>
static int launch_flash_fwd(const CUtensorMap& tq, const KvMaps& maps, const FlashFwdParams& p, cudaStream_t st) {
  using Cfg = FaFwdCfg<D>;
  static bool configured = false;
  auto kern = flash_fwd_kernel<D>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  dim3 grid(p.Hq, p.B, (p.Tq + kFaBlockQ - 1) / kFaBlockQ);
  kern<<<grid, kFaThreads, Cfg::kSmemBytes, st>>>(tq, maps, p);
  LT_LAUNCH_CHECK();
  return 0;
}

static int flash_fwd_common(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* o, float* lse, int B,
                            int Tq, int Tk, int Hq, int Hkv, int D, long long sq_b, long long sq_t, long long sk_b,
                            long long sk_t, long long sv_b, long long sv_t, long long so_b, long long so_t, float scale,
                            int causal, int cp_world, int cp_rank, int zigzag, void* stream) {
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || cp_world < 1 || cp_world > kFaMaxRanks) return -int(kStatusBadArgument);
  if (cp_world > 1 && zigzag && ((Tq / 2) % kFaBlockQ != 0 || (Tk / 2) % kFaBlockKV != 0)) return -int(kStatusBadArgument);
  if (cp_world > 1 && !zigzag && (Tq % kFaBlockQ != 0 || Tk % kFaBlockKV != 0)) return -int(kStatusBadArgument);
  if (B == 0 || Tq == 0) return 0;
  CUtensorMap tq;
  KvMaps maps;
  int r = encode_tmap_4d(&tq, q, 2, D, Hq, Tq, B, (uint64_t)D * 2, (uint64_t)sq_t * 2, (uint64_t)sq_b * 2, 64, 1, kFaBlockQ, 1, 1);
  if (r) return 1000 + r;
  for (int i = 0; i < kFaMaxRanks; ++i) {
    const int src = i < cp_world ? i : 0;
    r = encode_tmap_4d(&maps.k[i], k_ptrs[src], 2, D, Hkv, Tk, B, (uint64_t)D * 2, (uint64_t)sk_t * 2, (uint64_t)sk_b * 2, 64, 1,
                       kFaBlockKV, 1, 1);
    if (r) return 2000 + r;
    r = encode_tmap_4d(&maps.v[i], v_ptrs[src], 2, D, Hkv, Tk, B, (uint64_t)D * 2, (uint64_t)sv_t * 2, (uint64_t)sv_b * 2, 64, 1,
                       kFaBlockKV, 1, 1);
    if (r) return 3000 + r;
  }
  FlashFwdParams p{};
  p.O = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv;
  p.so_b = so_b; p.so_t = so_t;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.cp_world = cp_world; p.cp_rank = cp_rank; p.zigzag = zigzag;
  p.status = device_status_word();
  p.trace = g_fwd_trace;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return D == 64 ? launch_flash_fwd<64>(tq, maps, p, st) : launch_flash_fwd<128>(tq, maps, p, st);
}

}  // namespace lt

extern "C" {

// q: [B, Tq, Hq, D], k/v: [B, Tk, Hkv, D], o: [B, Tq, Hq, D]; strides in elements for the batch and time
// dimensions, heads are D apart, D contiguous.  lse: [B, Hq, Tq] fp32 (natural log).
// Debug aid: a device buffer of 16 int64 that the next forward launches fill with per-phase SM cycle counts of the
// CTA of the last query block of head 0 / batch 0 (warp 2, lane 0); nullptr switches it off.
void lt_flash_fwd_set_trace(void* buf) { lt::g_fwd_trace = static_cast<long long*>(buf); }

int lt_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int Hq, int Hkv,
                 int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t, long long sv_b, long long sv_t,
                 long long so_b, long long so_t, float scale, int causal, void* stream) {
  const void* ks[1] = {k};
  const void* vs[1] = {v};
  return lt::flash_fwd_common(q, ks, vs, o, lse, B, Tq, Tk, Hq, Hkv, D, sq_b, sq_t, sk_b, sk_t, sv_b, sv_t, so_b, so_t, scale,
                              causal, 1, 0, 0, stream);
}

// Context-parallel forward: k_ptrs[r] / v_ptrs[r] are rank r's KV shards [B, Tk, Hkv, D] (peer-mapped pointers, all with
// the same strides); the local queries attend to every rank's keys in one pass, the KV tiles of other ranks being
// read from peer memory by non-multicast TMA loads inside the kernel.
int lt_flash_fwd_cp(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* o, float* lse, int B, int Tq,
                    int Tk, int Hq, int Hkv, int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t,
                    long long sv_b, long long sv_t, long long so_b, long long so_t, float scale, int causal, int cp_world,
                    int cp_rank, int zigzag, void* stream) {
  return lt::flash_fwd_common(q, k_ptrs, v_ptrs, o, lse, B, Tq, Tk, Hq, Hkv, D, sq_b, sq_t, sk_b, sk_t, sv_b, sv_t, so_b, so_t,
                              scale, causal, cp_world, cp_rank, zigzag, stream);
}

}  // extern "C"
