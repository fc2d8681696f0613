// bf16 GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs computes one 256 x 256 output tile.
//
// With one CTA per 128 x 256 tile every SM pulls 48 KB of operands from L2 per 64-deep K block, which is more
// than an SM can take in while its tensor core runs flat out.  In a pair each CTA loads its own 128 rows of A and
// only HALF of the B tile (128 of the 256 columns); the MMA, issued by one thread of the even CTA, reads the B
// halves from both CTAs' shared memory and writes 128 accumulator rows into each CTA's tensor memory.  Operand
// traffic per SM drops to 32 KB per K block and the pipeline is 6 stages deep.
//
// Roles per CTA (192 threads): warp 0 TMA producer (both CTAs; the bytes of both are counted on the even CTA's
// full barrier), warp 1 TMEM allocation in both CTAs and MMA issue in the even CTA only, warps 2-5 epilogue of the
// CTA's own 128 rows (they release the accumulator buffer on the even CTA's barrier).
// The reference reaches its GEMMs through cuBLAS (src/backend/gpu_native/math/gemm.cu:3-189).
#pragma once
#include "gemm_sm100.cuh"

namespace lt {

constexpr int kPairBlockM = 256;   // rows of the pair's tile (128 per CTA)
constexpr int kPairBlockN = 256;   // columns of the pair's tile (each CTA stages 128 of them)
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kBlockM * kBlockK * 2 + (kPairBlockN / 2) * kBlockK * 2;   // 32 KB
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 512;
// Scatter epilogue (GEMM -> reduce-scatter): 8 KB of staging per epilogue warp behind the pipeline stages.
constexpr int kPairScatterStage = 32 * 128 * 2;          // 32 rows x 128 bf16 columns = two 128-byte-swizzled boxes
constexpr int kPairScatterSmemBytes = kPairStages * kPairStageBytes + 1024 + 4 * kPairScatterStage + 1024;   // stages, barriers, staging, alignment slack

// One tensor map per destination rank over its staging buffer [world * rows_per_rank, N] bf16, box 64 columns x 32
// rows, 128-byte swizzle: tiles travel to the owner as TMA stores (whole 128-byte lines over NVLink) instead of
// one 64-byte piece per lane.
struct ScatterMaps {
  CUtensorMap m[8];
};

int gemm_pair_mode();   // 0 never, 1 where the cost model prefers pairs, 2 always (set by lt_gemm_set_pair_mode)

// Tile counts of the pair kernel (256 x 256 tiles) in a GemmParams already filled by fill_tiles(p, 256).
inline void fill_pair_tiles(GemmParams& p) {
  p.m_blocks = (p.M + kPairBlockM - 1) / kPairBlockM;
  p.n_blocks = (p.N + kPairBlockN - 1) / kPairBlockN;
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.dp_tiles = p.num_tiles;
  p.group_m = 8;
}

// Parts per tile of the last, partly filled wave of pair tiles (1 = not cut).
inline int pair_tail_split(int num_tiles, int k_blocks, int pairs) {
  if (pairs <= 0 || num_tiles <= pairs) return 1;
  const int rem = num_tiles % pairs;
  if (rem == 0) return 1;
  // Measured: handing partial sums over through L2 costs about as much as a 32-block K loop, so only long-K GEMMs
  // (weight gradients, the down projection and its input gradient) come out ahead.
  if (k_blocks < 64) return 1;
  int s = pairs / rem;
  if (s > 4) s = 4;
  return s < 1 ? 1 : s;
}

// Time of the GEMM on CTA pairs in the unit of wave_cost (one wave of 128 x 256 tiles on every SM).
inline double pair_cost(int M, int N, int K, int sms, bool split_on) {
  const int tiles = ((M + kPairBlockM - 1) / kPairBlockM) * ((N + kPairBlockN - 1) / kPairBlockN);
  const int pairs = sms / 2 < tiles ? sms / 2 : tiles;
  const int s = split_on ? pair_tail_split(tiles, (K + kBlockK - 1) / kBlockK, pairs) : 1;
  const double waves = s > 1 ? double(tiles / pairs) + 1.0 / s + 0.06 : double((tiles + pairs - 1) / pairs);
  return waves * 0.88;   // a pair wave does the work of one single-CTA wave, measured 10-14 % faster (operand sharing)
}

// p.m_blocks / p.n_blocks / p.num_tiles count 256 x 256 tiles; everything else as in gemm_body.
// `gate(m_chunk, n_blk, kb, status)` and `done(m_chunk, n_blk)` are the hooks of gemm_body; m_chunk counts 128-row
// blocks (the rows one CTA of the pair loads and writes), n_blk counts 256-column blocks.  CTAs [0, cta_first) of
// the grid (an even number) belong to another role of a fused kernel.
template <int A_MAJOR, int B_MAJOR, int MMA_KIND = 0, class TileGate, class TileDone>   // MMA_KIND: see gemm_body
__device__ __forceinline__ void gemm_body_pair(const CUtensorMap* tmA, const CUtensorMap* tmB, const GemmParams& p,
                                               TileGate gate, TileDone done, int cta_first = 0,
                                               const ScatterMaps* scatter = nullptr) {
  constexpr int S = kPairStages;
  constexpr int kABytes = kBlockM * kBlockK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kPairStageBytes);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };            // used in the even CTA
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };     // one per CTA, signalled by the MMA commit
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); }; // one per CTA, signalled by the MMA commit
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };  // even CTA: 8 epilogue warps arrive
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = (cta_rank == 0);
  const int pair_id = (int(blockIdx.x) - cta_first) >> 1;
  const int pair_count = (int(gridDim.x) - cta_first) >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // both CTAs' barriers are initialised before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      for (int i = 0; ok && get_item(p, pair_id, pair_count, i, w); ++i) {
        int m_blk, n_blk;
        tile_coords(p, w.tile, m_blk, n_blk);
        const int m0 = m_blk * kPairBlockM + int(cta_rank) * kBlockM;
        const int n0 = n_blk * kPairBlockN + int(cta_rank) * (kPairBlockN / 2);
        for (int kl = w.kb0; kl < w.kb1; ++kl) {
          int kb = kl + p.k_rot;
          if (kb >= p.k_blocks) kb -= p.k_blocks;
          // (the odd CTA of the last pair may lie past M: it waits for the last real row block instead)
          if (!gate(min(m0, p.M - 1) / kBlockM, n_blk, kb, p.status)) { *abort_flag = 1; ok = false; break; }
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          const uint32_t fb = full_bar(stage);
          if (leader) mbar_expect_tx(fb, 2 * kPairStageBytes);   // this CTA's tiles and the odd CTA's
          const uint32_t a_dst = smem_base + stage * kPairStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          if (A_MAJOR == 0) {
            tma_load_2d_pair(a_dst, tmA, fb, kb * kBlockK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockM / 64; ++i)
              tma_load_2d_pair(a_dst + i * (64 * kBlockK * 2), tmA, fb, m0 + i * 64, kb * kBlockK);
          }
          if (B_MAJOR == 0) {
            tma_load_2d_pair(b_dst, tmB, fb, kb * kBlockK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < (kPairBlockN / 2) / 64; ++i)
              tma_load_2d_pair(b_dst + i * (64 * kBlockK * 2), tmB, fb, n0 + i * 64, kb * kBlockK);
          }
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = MMA_KIND == 4 ? make_idesc_e4m3(kPairBlockM, kPairBlockN)
                                           : make_idesc_f16(kPairBlockM, kPairBlockN, MMA_KIND == 2 ? 2 : (p.kind == 1 ? 0 : 1), A_MAJOR, B_MAJOR);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      for (int it = 0; ok && get_item(p, pair_id, pair_count, it, w); ++it) {
        const int buf = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aphase ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kPairBlockN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kPairStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t adesc = (A_MAJOR == 0) ? make_smem_desc_sw128(a_addr + k * (kUmmaK * 2), 16, 1024)
                                                  : make_smem_desc_sw128(a_addr + k * (kUmmaK * 128), 64 * kBlockK * 2, 1024);
            const uint64_t bdesc = (B_MAJOR == 0) ? make_smem_desc_sw128(b_addr + k * (kUmmaK * 2), 16, 1024)
                                                  : make_smem_desc_sw128(b_addr + k * (kUmmaK * 128), 64 * kBlockK * 2, 1024);
            if constexpr (MMA_KIND == 2) umma_tf32_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
            else if constexpr (MMA_KIND == 4) umma_e4m3_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
            else umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage), 3);   // the stage is free in both CTAs
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(buf), 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps per CTA, own 128 rows)
    const int quarter = warp & 3;
    int pend_m = -1, pend_n = 0;   // scatter epilogue: tile whose completion signal is still owed
    WorkItem w;
    for (int it = 0; get_item(p, pair_id, pair_count, it, w); ++it) {
      int m_blk, n_blk;
      tile_coords(p, w.tile, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      const bool got = mbar_wait(tfull_bar(buf), aphase, abort_flag, p.status, kStatusTimeoutTmemFull);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const int row = m_blk * kPairBlockM + int(cta_rank) * kBlockM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kPairBlockN;
      if (scatter != nullptr) {
        // GEMM -> reduce-scatter: this warp's 32 rows x 256 columns go to the rank that owns the rows as four TMA
        // stores of 32 x 64 bf16 (staged in shared memory, two boxes at a time).
        uint8_t* stg = smem + S * kPairStageBytes + 1024 + (warp - 2) * kPairScatterStage;
        const int row0 = m_blk * kPairBlockM + int(cta_rank) * kBlockM + quarter * 32;
        const bool live = row0 < p.M;
        const int owner = live ? row0 / p.rows_per_rank : 0;
        const int dst_row = p.src_rank * p.rows_per_rank + (row0 - owner * p.rows_per_rank);
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous stores have finished reading the staging area
          __syncwarp();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(t_addr + (hf * 4 + c) * 32, r);
            tmem_ld_wait();
            uint8_t* box = stg + (c >> 1) * (32 * 128) + lane * 128;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 w4;
              w4.x = pack_bf16x2(__uint_as_float(r[u * 8 + 0]) * p.alpha, __uint_as_float(r[u * 8 + 1]) * p.alpha);
              w4.y = pack_bf16x2(__uint_as_float(r[u * 8 + 2]) * p.alpha, __uint_as_float(r[u * 8 + 3]) * p.alpha);
              w4.z = pack_bf16x2(__uint_as_float(r[u * 8 + 4]) * p.alpha, __uint_as_float(r[u * 8 + 5]) * p.alpha);
              w4.w = pack_bf16x2(__uint_as_float(r[u * 8 + 6]) * p.alpha, __uint_as_float(r[u * 8 + 7]) * p.alpha);
              const int unit = ((c & 1) * 4 + u) ^ (lane & 7);
              *reinterpret_cast<uint4*>(box + unit * 16) = w4;
            }
          }
          if (hf == 1) {   // the accumulator buffer is in registers / shared memory: release it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_bar(buf), 0);
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (live) {
#pragma unroll
              for (int bx = 0; bx < 2; ++bx) {
                const int col = n_blk * kPairBlockN + hf * 128 + bx * 64;
                if (col < p.N) tma_store_2d(&scatter->m[owner], smem_u32(stg + bx * (32 * 128)), col, dst_row);
              }
            }
            tma_store_commit();   // always two groups per tile (possibly empty): the deferred signal counts on it
          }
        }
        // The owner is told about a tile only once its stores have completed at the owner, a round trip over NVLink.
        // Waiting for that here would put the round trip into every tile's epilogue, so the signal of a tile is sent
        // after the NEXT tile's stores have been committed (its own two groups are then the only ones that may
        // still be pending); the last tile's signal follows the loop.
        if (lane == 0) {
          if (pend_m >= 0) {
            tma_store_wait<2>();
            asm volatile("fence.proxy.async.global;" ::: "memory");
            done(pend_m, pend_n);   // a release at the scope the owner needs
          }
          pend_m = m_blk * (kPairBlockM / kBlockM) + int(cta_rank);
          pend_n = n_blk;
        }
        __syncwarp();
        continue;
      }
      // Split tail (see GemmParams): per split tile the workspace holds, for each other part, the two CTAs'
      // 128 x 256 fp32 accumulators as [chunk of 32 columns][group of 4 columns][row][4]; one flag per (tile, CTA, lane quarter).
      constexpr int kChunks = kPairBlockN / 32;
      auto part_base = [&](int part) {
        return p.sk_ws + ((long long)((w.slot * (p.sk_split - 1) + part) * 2 + int(cta_rank)) * kChunks) * (kBlockM * 32) +
               (quarter * 32 + lane) * 4;
      };
      unsigned* flag = p.sk_flags + (w.slot * 2 + int(cta_rank)) * 4 + quarter;
      if (w.split > 0) {
        float* ws = part_base(w.split - 1);
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_addr + c * 32, r);
          tmem_ld_wait();
          float4* dst = reinterpret_cast<float4*>(ws + (long long)c * (kBlockM * 32));
#pragma unroll
          for (int q = 0; q < 8; ++q)   // a warp writes 512 contiguous bytes per instruction (whole sectors)
            dst[q * kBlockM] = make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                                 __uint_as_float(r[q * 4 + 3]));
        }
        __threadfence();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster(tempty_bar(buf), 0);
          red_add_release_gpu(flag, 1u);
        }
        continue;
      }
      bool parts_ok = true;
      if (w.split == 0) {
        int okf = 1;
        if (lane == 0) {
          okf = wait_flag_ge_gpu(flag, uint32_t(p.sk_split - 1), p.status) ? 1 : 0;
          if (okf) *flag = 0u;   // the only waiter resets it for the next launch
        }
        parts_ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
      }
      if (!parts_ok) { *abort_flag = 1; break; }
      float4 pre[8];
      auto load_parts = [&](int c) {
#pragma unroll
        for (int q = 0; q < 8; ++q) pre[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < p.sk_split - 1; ++j) {
          const float4* src = reinterpret_cast<const float4*>(part_base(j) + (long long)c * (kBlockM * 32));
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 v = __ldcg(src + q * kBlockM);
            pre[q].x += v.x; pre[q].y += v.y; pre[q].z += v.z; pre[q].w += v.w;
          }
        }
      };
      if (w.split == 0) load_parts(0);
      auto add_parts = [&](uint32_t (&r)[32]) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          r[q * 4 + 0] = __float_as_uint(__uint_as_float(r[q * 4 + 0]) + pre[q].x);
          r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + pre[q].y);
          r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + pre[q].z);
          r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + pre[q].w);
        }
      };
      // two 32-column chunks per step: both tensor-memory loads are in flight before the first is consumed
#pragma unroll 1
      for (int c = 0; c < kChunks; c += 2) {
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(t_addr + c * 32, r0);
        tmem_ld_32x32(t_addr + (c + 1) * 32, r1);
        tmem_ld_wait();
        if (w.split == 0) {
          add_parts(r0);
          load_parts(c + 1);
          add_parts(r1);
          if (c + 2 < kChunks) load_parts(c + 2);
        }
        const int col0 = n_blk * kPairBlockN + c * 32;
        if (row < p.M && col0 < p.N) epilogue_store_chunk(p, row, col0, r0);
        if (row < p.M && col0 + 32 < p.N) epilogue_store_chunk(p, row, col0 + 32, r1);
      }
      done.fence();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(tempty_bar(buf), 0);
        done(m_blk * (kPairBlockM / kBlockM) + int(cta_rank), n_blk);
      }
    }
    if (scatter != nullptr && lane == 0 && pend_m >= 0) {
      tma_store_wait<0>();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      done(pend_m, pend_n);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // A bounded wait ran out: give copies that may still be in flight time to land before shared memory goes away.
    for (int spin = 0; spin < 20000; ++spin) __nanosleep(100);
  }
  cluster_sync_all();   // neither CTA frees tensor memory or leaves while its partner's MMAs or loads may touch it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace lt
