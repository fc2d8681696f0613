// FlashAttention backward for sm_100a: causal or full, grouped-query heads, bf16, head_dim 64 or 128.
//
// The reference backward recomputes S and P with cuBLAS into B*H*Tq*Tk fp32 scratch and runs five batched
// GEMMs plus two kernels (src/backend/gpu_native/nn/flash_attention.cu:395-713); GQA is only handled on the
// CPU by expanding K/V per head (src/ops/attention.cpp:88-175).  Here one CTA owns a block of 128 keys of one
// KV head and keeps dK and dV for it in tensor memory while it walks over every query head of the group and
// every query block that can see those keys:
//
//   S  = Q_i K^T        dP = dO_i V^T                 (tcgen05.mma into TMEM, 128 x 128 x D)
//   P  = exp2(S*c - lse),  dS = P * (dP - delta) * scale   (one query row per thread, written to shared
//                                                           memory in the swizzled operand layout)
//   dV += P^T dO_i      dK += dS^T Q_i                (A read M-major from the same P / dS tiles)
//   dQ_i = dS K         -> red.global.add into an fp32 accumulator, converted to bf16 by a last kernel
//
// delta = rowsum(O * dO) comes from a small pre-pass.  All waits are bounded (see common/ptx.cuh).
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kFbBlock = 128;
constexpr int kFbThreads = 384;   // warp 0 producer, warps 1 / 10 / 11 MMA issuers (S,dP / dV,dK / dQ), warps 2-9 compute
constexpr int kFbComputeThreads = 256;

constexpr int kFbMaxRanks = 8;
struct FlashBwdParams {
  // Per query-owning rank (index 0 only without context parallelism); peer-mapped pointers under CP:
  const float* lse[kFbMaxRanks];    // [B, Hq, Tq] natural log
  const float* delta[kFbMaxRanks];  // [B, Hq, Tq]
  float* dq_acc[kFbMaxRanks];       // [B, Tq, Hq, D] fp32, zero-initialised; remote ranks receive red.add over NVLink
  // Context parallelism: this rank's keys meet the queries of every rank; dK/dV stay local, dQ goes to its owner.
  int cp_world, cp_rank, zigzag;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;   // [B, Tk, Hkv, D] with strides sdk_b / sdk_t
  long long sdk_b, sdk_t;
  int B, Tq, Tk, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int* status;
  // Optional phase timing (nullptr: off): the CTA of key block 0 / head 0 / batch 0 adds the SM cycles its compute
  // warp 2 and its MMA thread spend in each phase to trace[0..15] and counts iterations in trace[15].
  long long* trace;
  int dbg;   // timing experiments only (results are wrong when non-zero): 1 = no bulk reduction, 2 = no staging either
};

struct QMaps {
  CUtensorMap q[kFbMaxRanks];
  CUtensorMap d_o[kFbMaxRanks];
};
struct QSeg {
  int n, owner, q0, qbase;   // a run of consecutive visible query blocks of one rank
};
constexpr int kFbMaxSegs = 2 * kFbMaxRanks;

template <int D>
struct FaBwdCfg {
  static constexpr int kTile = kFbBlock * D * 2;          // one 128 x D bf16 tile
  static constexpr int kPTile = kFbBlock * kFbBlock * 2;  // 128 x 128 bf16
  static constexpr int kStages = (D == 64) ? 2 : 1;       // Q / dO buffering
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kTile;
  static constexpr int kOffQ = 2 * kTile;
  static constexpr int kOffDO = kOffQ + kStages * kTile;
  static constexpr int kOffP = kOffDO + kStages * kTile;
  static constexpr int kOffDS = kOffP + kPTile;
  static constexpr int kOffBar = kOffDS + kPTile;
  static constexpr int kOffSeg = kOffBar + 128;
  // dQ tiles staged for TMA reductions into the fp32 accumulator (head_dim 64 only: with head_dim 128 shared memory
  // is full and the rows go out as red.global.add).  One 32-row x 32-column fp32 tile (4 KB, 128-byte swizzle) per
  // compute warp, reduced into global memory by ONE cp.reduce.async.bulk.tensor per warp and iteration: the copy
  // engine does the atomics, not the LSU, and it is given few, large operations.
  static constexpr bool kBulkDq = true;
  static constexpr int kDqTile = 32 * 128;                 // one 32-row x 32-column fp32 box
  static constexpr int kDqBoxes = D / 64;                  // boxes per warp: its 32 rows x D / 2 columns
  // head_dim 64: a staging area of its own.  head_dim 128: shared memory is full, so the staging area IS the P and dS
  // tiles (64 KB, free between the MMAs of one iteration and the exp phase of the next); a barrier among the compute
  // warps keeps the next exp phase from overwriting tiles a reduction is still reading.
  static constexpr bool kStageAliasesP = (D != 64);
  static constexpr int kOffDqStage = kStageAliasesP ? kOffP : ((kOffSeg + kFbMaxSegs * 16 + 16 + 1023) / 1024) * 1024;
  static constexpr int kSmemBytes = (kStageAliasesP ? kOffSeg + kFbMaxSegs * 16 + 16
                                                    : kOffDqStage + (kFbComputeThreads / 32) * kDqTile) + 1024;
  static constexpr int kColS = 0, kColDP = 128, kColDV = 256, kColDK = 256 + D;
  static constexpr int kColDQ = (D == 64) ? 384 : 0;  // D == 64: two buffers (384, 448); D == 128: aliases S
  // D == 64: dQ of iteration i is read one iteration later, right after S / dP of iteration i+1 arrive, when the
  // tensor pipe is idle (a tcgen05.ld issued while MMAs are queued waits behind them) and off the critical chain.
  static constexpr bool kDeferDq = (D == 64);
  static constexpr bool kDqAliasesS = (D != 64);
};

// delta[b,h,t] = sum_d O * dO ; D/8 threads per (b,t,h) row, 16 bytes each.
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                       float* __restrict__ delta, int B, int Tq, int Hq, int D, long long so_b,
                                       long long so_t, long long sdo_b, long long sdo_t) {
  const int tpr = D / 8;  // 8 or 16 threads per row
  const long long gid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long row = gid / tpr;
  const int sub = int(gid % tpr);
  const long long total = (long long)B * Tq * Hq;
  float s = 0.f;
  int h = 0, t = 0, b = 0;
  if (row < total) {
    h = int(row % Hq);
    t = int((row / Hq) % Tq);
    b = int(row / ((long long)Hq * Tq));
    const uint4 a = *reinterpret_cast<const uint4*>(O + b * so_b + t * so_t + (long long)h * D + sub * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + b * sdo_b + t * sdo_t + (long long)h * D + sub * 8);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = unpack_bf16x2(av[i]), y = unpack_bf16x2(gv[i]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = tpr / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (row < total && sub == 0) delta[((long long)b * Hq + h) * Tq + t] = s;
}

__global__ void flash_bwd_convert_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B, int Tq,
                                            int HD, long long sdq_b, long long sdq_t) {
  const long long n4 = (long long)B * Tq * HD / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 4;
    const int c = int(e % HD);
    const long long bt = e / HD;
    const int t = int(bt % Tq);
    const int b = int(bt / Tq);
    const float4 v = *reinterpret_cast<const float4*>(acc + e);
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + b * sdq_b + t * sdq_t + c) = o;
  }
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Asynchronous bulk reduction shared -> global: global[i] += shared[i] for `bytes` / 4 floats (16-byte aligned).
__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}
// Tiled TMA reduction shared -> global (fp32 add) of the box of `m` at coordinates (x, h, t, b).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, uint32_t smem_src, int x, int h, int t, int b) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_src), "r"(x), "r"(h), "r"(t), "r"(b) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(kFbThreads, 1)
flash_bwd_kernel(const __grid_constant__ QMaps qm, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDQ, const FlashBwdParams p) {
  using Cfg = FaBwdCfg<D>;
  constexpr int ST = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  const uint32_t bb = smem_u32(bars);
  const uint32_t kv_full = bb;
  auto qdo_full = [&](int s) { return bb + 8u * (1 + s); };
  auto qdo_empty = [&](int s) { return bb + 8u * (3 + s); };
  const uint32_t sdp_full = bb + 8u * 5;   // S and dP are in TMEM
  const uint32_t sdp_free = bb + 8u * 6;   // compute warps have read S and dP (one arrival per warp)
  const uint32_t pds_full = bb + 8u * 7;   // P and dS are in shared memory (one arrival per warp)
  const uint32_t pds_empty = bb + 8u * 8;  // the three MMAs that read P / dS have executed
  const uint32_t dq_full = bb + 8u * 9;    // dQ_i is in TMEM
  const uint32_t dq_free = bb + 8u * 10;   // compute warps have read dQ_i (one arrival per warp)
  const uint32_t dkv_full = bb + 8u * 11;  // all MMAs done
  const uint32_t dq_free1 = bb + 8u * 12;  // second dQ buffer (deferred-dQ flow)
  const uint32_t stg_free = bb + 8u * 13;  // every compute warp's dQ reduction has finished reading shared memory
  const uint32_t dq_full1 = bb + 8u * 14;  // dQ of odd iterations (deferred-dQ flow: one barrier per dQ buffer, so a
                                           // waiter can never be overtaken by two completions)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // x fastest in launch order: all (head, batch) pairs of key block 0 (seen by every query, the longest loop) first
  const int kv_blk = blockIdx.z, hkv = blockIdx.x, b = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int kv0 = kv_blk * kFbBlock;
  QSeg* segs = reinterpret_cast<QSeg*>(smem + Cfg::kOffSeg);
  int* per_head_s = reinterpret_cast<int*>(smem + Cfg::kOffSeg + kFbMaxSegs * 16);
  // global position of this block's first key
  int k_base;
  if (p.cp_world == 1) {
    k_base = kv0 - (p.Tk - p.Tq);   // expressed on the query axis: query i sees key j iff j - (Tk - Tq) <= i
  } else if (p.zigzag) {
    const int hk = p.Tk / 2;
    k_base = kv0 < hk ? p.cp_rank * hk + kv0 : (2 * p.cp_world - 1 - p.cp_rank) * hk + (kv0 - hk);
  } else {
    k_base = p.cp_rank * p.Tk + kv0;
  }
  if (threadIdx.x == 0) {
    // query blocks that see these keys, as runs per owning rank (own rank first)
    int ns = 0, total = 0;
    for (int i = 0; i < p.cp_world; ++i) {
      const int o = (p.cp_rank + i) % p.cp_world;
      const int parts = (p.cp_world > 1 && p.zigzag) ? 2 : 1;
      for (int h2 = 0; h2 < parts; ++h2) {
        int q0s, qbase, nb;
        if (parts == 2) {
          const int hq = p.Tq / 2;
          q0s = h2 * hq;
          qbase = h2 == 0 ? o * hq : (2 * p.cp_world - 1 - o) * hq;
          nb = hq / kFbBlock;
        } else {
          q0s = 0;
          qbase = p.cp_world > 1 ? o * p.Tq : 0;
          nb = (p.Tq + kFbBlock - 1) / kFbBlock;
        }
        int skip = 0;
        if (p.causal) {
          const int first_q = k_base - qbase;   // first query position (relative to the run) that sees key k_base
          skip = first_q <= 0 ? 0 : first_q / kFbBlock;
        }
        if (nb > skip) {
          segs[ns] = QSeg{nb - skip, o, q0s + skip * kFbBlock, qbase + skip * kFbBlock};
          ++ns;
          total += nb - skip;
        }
      }
    }
    for (int i = ns; i < kFbMaxSegs; ++i) segs[i] = QSeg{0, 0, 0, 0};
    *per_head_s = total;
  }
  __syncthreads();
  const int per_head = *per_head_s;
  const int n_iter = per_head * G;
  auto locate = [&](int j, int& owner, int& q0, int& qbase) {
    int sidx = 0;
    while (sidx < kFbMaxSegs - 1 && j >= segs[sidx].n) { j -= segs[sidx].n; ++sidx; }
    owner = segs[sidx].owner;
    q0 = segs[sidx].q0 + j * kFbBlock;
    qbase = segs[sidx].qbase + j * kFbBlock;
  };

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(qdo_full(s), 1); mbar_init(qdo_empty(s), 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_free, kFbComputeThreads / 32);
    mbar_init(pds_full, kFbComputeThreads / 32); mbar_init(pds_empty, 2);   // the dV/dK and the dQ issuer release P / dS
    mbar_init(dq_full, 1); mbar_init(dq_full1, 1); mbar_init(dq_free, kFbComputeThreads / 32); mbar_init(dq_free1, kFbComputeThreads / 32);
    mbar_init(stg_free, kFbComputeThreads / 32);
    mbar_init(dkv_full, 2);   // the dV/dK and the dQ issuer have drained
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&qm.q[p.cp_rank]); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&qm.d_o[p.cp_rank]);
    tma_prefetch_desc(&tmDQ);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::kTile);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        tma_load_4d(sbase + Cfg::kOffK + c * (kFbBlock * 128), &tmK, kv_full, c * 64, hkv, kv0, b);
        tma_load_4d(sbase + Cfg::kOffV + c * (kFbBlock * 128), &tmV, kv_full, c * 64, hkv, kv0, b);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % ST;
        const uint32_t par = (it / ST) & 1;
        const int h = hkv * G + it / per_head;
        int owner, q0, qbase;
        locate(it % per_head, owner, q0, qbase);
        if (!mbar_wait(qdo_empty(s), par ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) break;
        mbar_expect_tx(qdo_full(s), 2 * Cfg::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          tma_load_4d(sbase + Cfg::kOffQ + s * Cfg::kTile + c * (kFbBlock * 128), &qm.q[owner], qdo_full(s), c * 64, h, q0, b);
          tma_load_4d(sbase + Cfg::kOffDO + s * Cfg::kTile + c * (kFbBlock * 128), &qm.d_o[owner], qdo_full(s), c * 64, h, q0, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- first MMA issuer: S = Q K^T, dP = dO V^T
    // (as far ahead as the S / dP columns of tensor memory allow: they are free once the compute warps have loaded them)
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_sd = make_idesc_f16(128, 128, 1, 0, 0);  // S, dP: A K-major, B K-major
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kStatusTimeoutFull);
      const uint32_t ka = sbase + Cfg::kOffK, va = sbase + Cfg::kOffV;
      const bool tr = p.trace != nullptr && kv_blk == 0 && hkv == 0 && b == 0;
      long long tm[4] = {0, 0, 0, 0};
      for (int it = 0; ok && it < n_iter; ++it) {
        const int s = it % ST;
        const uint32_t par = (it / ST) & 1;
        const uint32_t ipar = it & 1;
        const uint32_t qa = sbase + Cfg::kOffQ + s * Cfg::kTile;
        const uint32_t doa = sbase + Cfg::kOffDO + s * Cfg::kTile;
        long long c0 = tr ? clock64() : 0;
        if (!mbar_wait(qdo_full(s), par, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
        if (tr) { const long long c1 = clock64(); tm[0] += c1 - c0; c0 = c1; }
        if (!mbar_wait(sdp_free, ipar ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
        if (tr) { const long long c1 = clock64(); tm[1] += c1 - c0; c0 = c1; }
        if (Cfg::kDqAliasesS) {
          if (!mbar_wait(dq_free, ipar ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_base + Cfg::kColS, make_smem_desc_sw128(qa + off, 16, 1024),
                      make_smem_desc_sw128(ka + off, 16, 1024), idesc_sd, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16_ss(tmem_base + Cfg::kColDP, make_smem_desc_sw128(doa + off, 16, 1024),
                      make_smem_desc_sw128(va + off, 16, 1024), idesc_sd, k > 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
      }
      if (tr) {
        // MMA thread: wait for Q/dO, for S/dP to be read, for P/dS
        p.trace[8] = tm[0]; p.trace[9] = tm[1]; p.trace[10] = tm[2];
      }
    }
  } else if (warp == 11) {
    // ---------------------------------------------------------------- third MMA issuer: dQ_i = dS K
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_dq = make_idesc_f16(128, D, 1, 0, 1);    // A K-major, B N-major
      const uint32_t ka = sbase + Cfg::kOffK, dsa = sbase + Cfg::kOffDS;
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kStatusTimeoutFull);
      for (int it = 0; ok && it < n_iter; ++it) {
        const uint32_t ipar = it & 1;
        if (!mbar_wait(pds_full, ipar, abort_flag, p.status, kStatusTimeoutTmemFull)) break;
        if (!Cfg::kDqAliasesS) {
          // dQ buffer it & 1 was last used by iteration it - 2
          if (!mbar_wait((it & 1) ? dq_free1 : dq_free, ((uint32_t(it) >> 1) & 1u) ^ 1u, abort_flag, p.status,
                         kStatusTimeoutTmemEmpty)) break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kFbBlock / 16; ++k) {   // K dimension = the 128 keys
          const uint64_t adesc = make_smem_desc_sw128(dsa + (k / 4) * (128 * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(ka + k * (16 * 128), 128 * 128, 1024);
          umma_f16_ss(tmem_base + Cfg::kColDQ + (Cfg::kDeferDq ? (it & 1) * D : 0), adesc, bdesc, idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(pds_empty);
        umma_commit((Cfg::kDeferDq && (it & 1)) ? dq_full1 : dq_full);
        if (it == n_iter - 1) umma_commit(dkv_full);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- second MMA issuer: dV += P^T dO, dK += dS^T Q
    // Issuing a tcgen05.mma costs its thread on the order of a hundred cycles whatever the tile width, and in this
    // kernel the issue time sits on the critical chain (the exp phase of the next iteration waits for all of them):
    // the 16 dV / dK MMAs of an iteration go out from this thread while warp 1 issues dQ and the next S / dP.
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_kv = make_idesc_f16(128, D, 1, 1, 1);    // A M-major, B N-major
      const uint32_t pa = sbase + Cfg::kOffP, dsa = sbase + Cfg::kOffDS;
      for (int it = 0; it < n_iter; ++it) {
        const int s = it % ST;
        const uint32_t ipar = it & 1;
        const uint32_t qa = sbase + Cfg::kOffQ + s * Cfg::kTile;
        const uint32_t doa = sbase + Cfg::kOffDO + s * Cfg::kTile;
        // P / dS ready implies Q / dO of this stage are in shared memory (S and dP were computed from them)
        if (!mbar_wait(pds_full, ipar, abort_flag, p.status, kStatusTimeoutTmemFull)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kFbBlock / 16; ++k) {   // K dimension = the 128 query rows, 16 rows per instruction
          const uint32_t koff = k * (16 * 128);
          umma_f16_ss(tmem_base + Cfg::kColDV, make_smem_desc_sw128(pa + koff, 128 * 128, 1024),
                      make_smem_desc_sw128(doa + koff, 128 * 128, 1024), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kFbBlock / 16; ++k) {
          const uint32_t koff = k * (16 * 128);
          umma_f16_ss(tmem_base + Cfg::kColDK, make_smem_desc_sw128(dsa + koff, 128 * 128, 1024),
                      make_smem_desc_sw128(qa + koff, 128 * 128, 1024), idesc_kv, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(qdo_empty(s));
        umma_commit(pds_empty);
        if (it == n_iter - 1) umma_commit(dkv_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps
    // Two warps share each TMEM lane quarter (a warp may only touch lanes 32*(warp%4)..+31); they split the columns.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    bool ok = true;
    const bool tr = p.trace != nullptr && kv_blk == 0 && hkv == 0 && b == 0 && warp == 2 && lane == 0;
    long long tc[6] = {0, 0, 0, 0, 0, 0};
    // Row statistics are fetched one iteration ahead (the global-load latency is off the chain); the position of an
    // iteration (query head, block within the head) is advanced with counters, not divisions.
    const bool single = (p.cp_world == 1);
    const float* lse0 = p.lse[0];
    const float* delta0 = p.delta[0];
    float* dq0 = p.dq_acc[0];
    auto fetch_stats = [&](int hh, int jj, float& lse_raw, float& dl) {
      lse_raw = 0.f; dl = 0.f;
      if (hh >= G) return;
      const int h = hkv * G + hh;
      int owner, q0, qbase;
      locate(jj, owner, q0, qbase);
      const int q_idx = q0 + row;
      if (q_idx < p.Tq) {
        const long long si = ((long long)b * p.Hq + h) * p.Tq + q_idx;
        // (indexing the pointer arrays of the kernel parameters with a run-time rank makes the compiler copy them to
        // local memory: the single-rank case reads element 0 directly)
        lse_raw = single ? lse0[si] : p.lse[owner][si];
        dl = single ? delta0[si] : p.delta[owner][si];
      }
    };
    float lse_next, dlt_next;
    int hh_next = 0, jj_next = 0;   // position of the iteration whose statistics are in lse_next / dlt_next
    fetch_stats(n_iter > 0 ? 0 : G, 0, lse_next, dlt_next);
    bool dq_pending = false;   // this thread has a bulk reduction in flight that reads its staging piece
    // This warp's 32 x (D / 2) piece of one dQ tile: TMEM -> registers -> global accumulator; the TMEM buffer is
    // released as soon as the values are in registers.
    auto emit_dq = [&](int buf, float* dq_row, bool valid, bool local, int h_, int q0_) {
      if (Cfg::kBulkDq && local) {
        uint8_t* tile = smem + Cfg::kOffDqStage + (warp - 2) * (Cfg::kDqBoxes * Cfg::kDqTile);
        if (!Cfg::kStageAliasesP && dq_pending) {   // the previous reduction has finished reading the tile
          if (lane == 0) bulk_wait_read0();
          __syncwarp();
        }
#pragma unroll
        for (int bx = 0; bx < Cfg::kDqBoxes; ++bx) {
          uint32_t dq[32];
          tmem_ld_32x32(tmem_base + lane_base + Cfg::kColDQ + buf * D + (half * Cfg::kDqBoxes + bx) * 32, dq);
          tmem_ld_wait();
          if (bx == Cfg::kDqBoxes - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(buf ? dq_free1 : dq_free);
          }
          if (p.dbg >= 2) continue;
#pragma unroll
          for (int u = 0; u < 8; ++u)   // row `lane` of the box, 16-byte units swizzled like the tensor map expects
            *reinterpret_cast<uint4*>(tile + bx * Cfg::kDqTile + lane * 128 + ((u ^ (lane & 7)) * 16)) =
                make_uint4(dq[u * 4], dq[u * 4 + 1], dq[u * 4 + 2], dq[u * 4 + 3]);
        }
        if (p.dbg >= 2) return;
        fence_proxy_async();
        __syncwarp();
        dq_pending = false;
        if (p.dbg == 0) {
          if (lane == 0) {
#pragma unroll
            for (int bx = 0; bx < Cfg::kDqBoxes; ++bx)   // rows past Tq are clipped by the copy engine
              tma_reduce_add_4d(&tmDQ, smem_u32(tile + bx * Cfg::kDqTile), (half * Cfg::kDqBoxes + bx) * 32, h_,
                                q0_ + quarter * 32, b);
            bulk_commit();
          }
          dq_pending = true;
        }
      } else {
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t dq[32];
          tmem_ld_32x32(tmem_base + lane_base + Cfg::kColDQ + buf * D + c * 32, dq);
          tmem_ld_wait();
          if (valid) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              red_add_v4(dq_row + c * 32 + u * 4, __uint_as_float(dq[u * 4]), __uint_as_float(dq[u * 4 + 1]),
                         __uint_as_float(dq[u * 4 + 2]), __uint_as_float(dq[u * 4 + 3]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(buf ? dq_free1 : dq_free);
      }
    };
    float* prev_row = nullptr;   // deferred-dQ flow: where the previous iteration's dQ row goes
    bool prev_valid = false, prev_local = true;
    int prev_h = 0, prev_q0 = 0;
    for (int it = 0; it < n_iter; ++it) {
      long long c0 = tr ? clock64() : 0;
      const uint32_t ipar = it & 1;
      const int h = hkv * G + hh_next;
      int owner, q0, qbase;
      locate(jj_next, owner, q0, qbase);
      const int q_idx = q0 + row;
      const bool q_valid = q_idx < p.Tq;
      const float lse2 = lse_next * 1.4426950408889634f, dlt = dlt_next;
      if (++jj_next == per_head) { jj_next = 0; ++hh_next; }
      fetch_stats(hh_next, jj_next, lse_next, dlt_next);
      // last visible key (index local to this rank's KV) for this query row
      const int limit = p.causal ? min(kv0 + (qbase + row - k_base), p.Tk - 1) : (p.Tk - 1);
      if (tr) { const long long c1 = clock64(); tc[0] += c1 - c0; c0 = c1; }   // lse / delta loads issued, index math
      ok = __all_sync(0xffffffffu, mbar_wait(sdp_full, ipar, abort_flag, p.status, kStatusTimeoutTmemFull));
      if (!ok) break;
      if (tr) { const long long c1 = clock64(); tc[1] += c1 - c0; c0 = c1; }   // waiting for S / dP
      // P / dS tiles are free once the MMAs of the previous iteration have executed.
      ok = __all_sync(0xffffffffu, mbar_wait(pds_empty, ipar ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty));
      if (!ok) break;
      if (Cfg::kStageAliasesP && it > 0) {
        // ... and once every warp's dQ reduction of the previous iteration has finished reading them
        if (lane == 0) {
          if (dq_pending) bulk_wait_read0();
          mbar_arrive(stg_free);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(stg_free, uint32_t(it - 1) & 1u, abort_flag, p.status, kStatusTimeoutLocalFlag));
        if (!ok) break;
      }
      if (tr) { const long long c1 = clock64(); tc[2] += c1 - c0; c0 = c1; }   // waiting for the P / dS tiles
      tc_fence_after();
      uint8_t* prow = smem + Cfg::kOffP + (row >> 3) * 1024 + (row & 7) * 128;
      uint8_t* dsrow = smem + Cfg::kOffDS + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32(tmem_base + lane_base + Cfg::kColS + c * 32, sv);
        tmem_ld_32x32(tmem_base + lane_base + Cfg::kColDP + c * 32, dp);
        tmem_ld_wait();
        if (c == 2 * half + 1) {   // S / dP are in registers: the next iteration's score products may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sdp_free);
        }
        const bool live = q_valid && lse2 != -INFINITY;
        const float dlt_s = dlt * p.scale;
        if (live && kv0 + c * 32 + 31 <= limit) {   // every column of the chunk is visible: no per-element test
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pv = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse2));
            const float ds = pv * fmaf(__uint_as_float(dp[i]), p.scale, -dlt_s);
            sv[i] = __float_as_uint(pv);
            dp[i] = __float_as_uint(ds);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kv_idx = kv0 + c * 32 + i;
            float pv = 0.f;
            if (live && kv_idx <= limit) pv = ex2_approx(fmaf(__uint_as_float(sv[i]), p.scale_log2, -lse2));
            const float ds = pv * fmaf(__uint_as_float(dp[i]), p.scale, -dlt_s);
            sv[i] = __float_as_uint(pv);
            dp[i] = __float_as_uint(ds);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          uint4 w, z;
          w.x = pack_bf16x2(__uint_as_float(sv[u * 8 + 0]), __uint_as_float(sv[u * 8 + 1]));
          w.y = pack_bf16x2(__uint_as_float(sv[u * 8 + 2]), __uint_as_float(sv[u * 8 + 3]));
          w.z = pack_bf16x2(__uint_as_float(sv[u * 8 + 4]), __uint_as_float(sv[u * 8 + 5]));
          w.w = pack_bf16x2(__uint_as_float(sv[u * 8 + 6]), __uint_as_float(sv[u * 8 + 7]));
          z.x = pack_bf16x2(__uint_as_float(dp[u * 8 + 0]), __uint_as_float(dp[u * 8 + 1]));
          z.y = pack_bf16x2(__uint_as_float(dp[u * 8 + 2]), __uint_as_float(dp[u * 8 + 3]));
          z.z = pack_bf16x2(__uint_as_float(dp[u * 8 + 4]), __uint_as_float(dp[u * 8 + 5]));
          z.w = pack_bf16x2(__uint_as_float(dp[u * 8 + 6]), __uint_as_float(dp[u * 8 + 7]));
          const int col16 = c * 4 + u;
          const int chunk = col16 >> 3;
          const int unit = (col16 & 7) ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + chunk * (128 * 128) + unit * 16) = w;
          *reinterpret_cast<uint4*>(dsrow + chunk * (128 * 128) + unit * 16) = z;
        }
      }
      // one arrival per warp: 256 same-address arrivals on a shared-memory barrier serialise
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (tr) { const long long c1 = clock64(); tc[3] += c1 - c0; c0 = c1; }   // exp / dS / stores to shared memory
      if (Cfg::kDeferDq) {
        // While the tensor core works on dV / dK / dQ of this iteration and S / dP of the next, write out dQ of the
        // PREVIOUS iteration: it is complete (S / dP of this iteration were committed after it), and its transfer
        // TMEM -> registers -> shared memory -> TMA reduction is off the critical chain here.
        if (it > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(((it - 1) & 1) ? dq_full1 : dq_full, (uint32_t(it - 1) >> 1) & 1u, abort_flag,
                                                 p.status, kStatusTimeoutTmemFull));
          if (!ok) break;
          tc_fence_after();
          emit_dq((it - 1) & 1, prev_row, prev_valid, prev_local, prev_h, prev_q0);
          if (tr) { const long long c1 = clock64(); tc[5] += c1 - c0; c0 = c1; }
        }
        prev_row = (single ? dq0 : p.dq_acc[owner]) + (((long long)b * p.Tq + q_idx) * p.Hq + h) * D;
        prev_valid = q_valid;
        prev_local = (owner == p.cp_rank);
        prev_h = h; prev_q0 = q0;
        continue;
      }
      // dQ_i
      ok = __all_sync(0xffffffffu, mbar_wait(dq_full, ipar, abort_flag, p.status, kStatusTimeoutTmemFull));
      if (!ok) break;
      if (tr) { const long long c1 = clock64(); tc[4] += c1 - c0; c0 = c1; }   // waiting for dQ
      if (Cfg::kStageAliasesP) {
        // the staging area is the P / dS tiles: the dV / dK MMAs of the other issuer must be done with them too
        ok = __all_sync(0xffffffffu, mbar_wait(pds_empty, ipar, abort_flag, p.status, kStatusTimeoutTmemEmpty));
        if (!ok) break;
      }
      tc_fence_after();
      emit_dq(0, (single ? dq0 : p.dq_acc[owner]) + (((long long)b * p.Tq + q_idx) * p.Hq + h) * D, q_valid,
              owner == p.cp_rank, h, q0);
      if (tr) { const long long c1 = clock64(); tc[5] += c1 - c0; c0 = c1; }   // dQ read + reduction
    }
    if (tr) {
      for (int i = 0; i < 6; ++i) p.trace[i] = tc[i];
      p.trace[15] = n_iter;
    }
    // ---------------------------------------------------------------- dK / dV epilogue (row = key index)
    if (ok && n_iter > 0) ok = __all_sync(0xffffffffu, mbar_wait(dkv_full, 0, abort_flag, p.status, kStatusTimeoutTmemFull));
    if (Cfg::kDeferDq && ok && n_iter > 0) {
      tc_fence_after();
      emit_dq((n_iter - 1) & 1, prev_row, prev_valid, prev_local, prev_h, prev_q0);   // dQ of the last iteration
    }
    if (dq_pending && lane == 0) bulk_wait_all0();   // shared memory must outlive the reductions that read it
    if (ok) {
      if (n_iter > 0) tc_fence_after();
      const int kv_idx = kv0 + row;
      __nv_bfloat16* dk_row = p.dK + b * p.sdk_b + (long long)kv_idx * p.sdk_t + (long long)hkv * D;
      __nv_bfloat16* dv_row = p.dV + b * p.sdk_b + (long long)kv_idx * p.sdk_t + (long long)hkv * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t a[32], g[32];
        if (n_iter > 0) {
          tmem_ld_32x32(tmem_base + lane_base + Cfg::kColDK + c * 32, a);
          tmem_ld_32x32(tmem_base + lane_base + Cfg::kColDV + c * 32, g);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0u; g[i] = 0u; }
        }
        if (kv_idx < p.Tk) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 w, z;
            w.x = pack_bf16x2(__uint_as_float(a[u * 8 + 0]), __uint_as_float(a[u * 8 + 1]));
            w.y = pack_bf16x2(__uint_as_float(a[u * 8 + 2]), __uint_as_float(a[u * 8 + 3]));
            w.z = pack_bf16x2(__uint_as_float(a[u * 8 + 4]), __uint_as_float(a[u * 8 + 5]));
            w.w = pack_bf16x2(__uint_as_float(a[u * 8 + 6]), __uint_as_float(a[u * 8 + 7]));
            z.x = pack_bf16x2(__uint_as_float(g[u * 8 + 0]), __uint_as_float(g[u * 8 + 1]));
            z.y = pack_bf16x2(__uint_as_float(g[u * 8 + 2]), __uint_as_float(g[u * 8 + 3]));
            z.z = pack_bf16x2(__uint_as_float(g[u * 8 + 4]), __uint_as_float(g[u * 8 + 5]));
            z.w = pack_bf16x2(__uint_as_float(g[u * 8 + 6]), __uint_as_float(g[u * 8 + 7]));
            *reinterpret_cast<uint4*>(dk_row + c * 32 + u * 8) = w;
            *reinterpret_cast<uint4*>(dv_row + c * 32 + u * 8) = z;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int spin = 0; spin < 2000; ++spin) __nanosleep(100);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D>
static int launch_flash_bwd(const QMaps& qm, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdq,
                            const FlashBwdParams& p, cudaStream_t st) {
  using Cfg = FaBwdCfg<D>;
  static bool configured = false;
  auto kern = flash_bwd_kernel<D>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  dim3 grid(p.Hkv, p.B, (p.Tk + kFbBlock - 1) / kFbBlock);
  kern<<<grid, kFbThreads, Cfg::kSmemBytes, st>>>(qm, tk, tv, tdq, p);
  LT_LAUNCH_CHECK();
  return 0;
}

static int bwd_delta(const void* o, const void* d_o, float* delta, int B, int Tq, int Hq, int D, long long so_b, long long so_t,
                     long long sdo_b, long long sdo_t, cudaStream_t st) {
  const long long rows = (long long)B * Tq * Hq;
  const int threads = 256;
  const long long blocks = (rows * (D / 8) + threads - 1) / threads;
  flash_bwd_delta_kernel<<<(unsigned)blocks, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(o),
                                                               static_cast<const __nv_bfloat16*>(d_o), delta, B, Tq, Hq, D, so_b,
                                                               so_t, sdo_b, sdo_t);
  LT_LAUNCH_CHECK();
  return 0;
}

static int bwd_convert(const float* dq_acc, void* dq, int B, int Tq, int Hq, int D, long long sdq_b, long long sdq_t,
                       cudaStream_t st) {
  const long long n4 = (long long)B * Tq * Hq * D / 4;
  long long blocks = (n4 + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  flash_bwd_convert_dq_kernel<<<(unsigned)blocks, 256, 0, st>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), B, Tq, Hq * D, sdq_b, sdq_t);
  LT_LAUNCH_CHECK();
  return 0;
}

// Main kernel.  q/d_o/lse/delta/dq_acc are given per query-owning rank (cp_world entries; peer-mapped under CP).
static long long* g_bwd_trace = nullptr;

static int bwd_main(const void* const* q_ptrs, const void* k, const void* v, const void* const* do_ptrs,
                    const float* const* lse_ptrs, const float* const* delta_ptrs, float* const* dq_acc_ptrs, void* dk, void* dv,
                    int B, int Tq, int Tk, int Hq, int Hkv, int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t,
                    long long sv_b, long long sv_t, long long sdo_b, long long sdo_t, long long sdk_b, long long sdk_t,
                    float scale, int causal, int cp_world, int cp_rank, int zigzag, cudaStream_t st) {
  if (cp_world < 1 || cp_world > kFbMaxRanks) return -int(kStatusBadArgument);
  if (cp_world > 1 && zigzag && ((Tq / 2) % kFbBlock != 0 || (Tk / 2) % kFbBlock != 0)) return -int(kStatusBadArgument);
  if (cp_world > 1 && !zigzag && (Tq % kFbBlock != 0 || Tk % kFbBlock != 0)) return -int(kStatusBadArgument);
  QMaps qm;
  CUtensorMap tk, tv;
  int r;
  for (int i = 0; i < kFbMaxRanks; ++i) {
    const int src = i < cp_world ? i : 0;
    r = encode_tmap_4d(&qm.q[i], q_ptrs[src], 2, D, Hq, Tq, B, (uint64_t)D * 2, (uint64_t)sq_t * 2, (uint64_t)sq_b * 2, 64, 1,
                       kFbBlock, 1, 1);
    if (r) return 1000 + r;
    r = encode_tmap_4d(&qm.d_o[i], do_ptrs[src], 2, D, Hq, Tq, B, (uint64_t)D * 2, (uint64_t)sdo_t * 2, (uint64_t)sdo_b * 2, 64,
                       1, kFbBlock, 1, 1);
    if (r) return 4000 + r;
  }
  r = encode_tmap_4d(&tk, k, 2, D, Hkv, Tk, B, (uint64_t)D * 2, (uint64_t)sk_t * 2, (uint64_t)sk_b * 2, 64, 1, kFbBlock, 1, 1);
  if (r) return 2000 + r;
  r = encode_tmap_4d(&tv, v, 2, D, Hkv, Tk, B, (uint64_t)D * 2, (uint64_t)sv_t * 2, (uint64_t)sv_b * 2, 64, 1, kFbBlock, 1, 1);
  if (r) return 3000 + r;
  FlashBwdParams p{};
  for (int i = 0; i < cp_world; ++i) {
    p.lse[i] = lse_ptrs[i];
    p.delta[i] = delta_ptrs[i];
    p.dq_acc[i] = dq_acc_ptrs[i];
  }
  p.cp_world = cp_world; p.cp_rank = cp_rank; p.zigzag = zigzag;
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.sdk_b = sdk_b; p.sdk_t = sdk_t;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = device_status_word();
  p.trace = g_bwd_trace;
  p.dbg = 0;
  // fp32 dQ accumulator of this rank, [B, Tq, Hq, D]: boxes of 32 rows x 32 columns (128 bytes, swizzled)
  CUtensorMap tdq;
  r = encode_tmap_4d(&tdq, dq_acc_ptrs[cp_rank], 4, D, Hq, Tq, B, (uint64_t)D * 4, (uint64_t)Hq * D * 4,
                     (uint64_t)Tq * Hq * D * 4, 32, 1, 32, 1, 1);
  if (r) return 5000 + r;
  return (D == 64) ? launch_flash_bwd<64>(qm, tk, tv, tdq, p, st) : launch_flash_bwd<128>(qm, tk, tv, tdq, p, st);
}

}  // namespace lt

extern "C" {

// Shapes as lt_flash_fwd.  delta: scratch [B, Hq, Tq] fp32.  dq_acc: scratch [B, Tq, Hq, D] fp32, must be zero.
// dk and dv share the strides sdk_b / sdk_t.
// Debug aid: a device buffer of 16 int64 that the next backward launches fill with per-phase SM cycle counts of one
// CTA (see FlashBwdParams::trace); nullptr switches it off.
void lt_flash_bwd_set_trace(void* buf) { lt::g_bwd_trace = static_cast<long long*>(buf); }

int lt_flash_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o, void* dq,
                 void* dk, void* dv, float* delta, float* dq_acc, int B, int Tq, int Tk, int Hq, int Hkv, int D,
                 long long sq_b, long long sq_t, long long sk_b, long long sk_t, long long sv_b, long long sv_t,
                 long long so_b, long long so_t, long long sdo_b, long long sdo_t, long long sdq_b, long long sdq_t,
                 long long sdk_b, long long sdk_t, float scale, int causal, void* stream) {
  using namespace lt;
  if ((D != 64 && D != 128) || Hq % Hkv != 0) return -int(kStatusBadArgument);
  if (B == 0 || Tq == 0 || Tk == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = bwd_delta(o, d_o, delta, B, Tq, Hq, D, so_b, so_t, sdo_b, sdo_t, st);
  if (rc) return rc;
  const void* qs[1] = {q};
  const void* dos[1] = {d_o};
  const float* lses[1] = {lse};
  const float* deltas[1] = {delta};
  float* accs[1] = {dq_acc};
  rc = bwd_main(qs, k, v, dos, lses, deltas, accs, dk, dv, B, Tq, Tk, Hq, Hkv, D, sq_b, sq_t, sk_b, sk_t, sv_b, sv_t, sdo_b, sdo_t,
                sdk_b, sdk_t, scale, causal, 1, 0, 0, st);
  if (rc) return rc;
  return bwd_convert(dq_acc, dq, B, Tq, Hq, D, sdq_b, sdq_t, st);
}

// Context-parallel backward in three stream-ordered phases; the caller crosses a rank barrier between them.
//   phase 0: delta = rowsum(O * dO) of the local queries (into symmetric memory); the caller also zeroes dq_acc.
//   phase 1: main kernel - this rank's keys against every rank's queries: Q / dO tiles by TMA from peer memory, lse / delta
//            by peer loads, dK / dV accumulated locally, dQ added to the owner's fp32 accumulator with red.add over NVLink.
//   phase 2: dq = bf16(dq_acc) once every peer's phase 1 is complete.
int lt_flash_bwd_cp(int phase, const void* const* q_ptrs, const void* k, const void* v, const void* o, const void* const* do_ptrs,
                    const float* const* lse_ptrs, const float* const* delta_ptrs, float* const* dq_acc_ptrs, void* dq, void* dk,
                    void* dv, int B, int Tq, int Tk, int Hq, int Hkv, int D, long long sq_b, long long sq_t, long long sk_b,
                    long long sk_t, long long sv_b, long long sv_t, long long so_b, long long so_t, long long sdo_b,
                    long long sdo_t, long long sdq_b, long long sdq_t, long long sdk_b, long long sdk_t, float scale, int causal,
                    int cp_world, int cp_rank, int zigzag, void* stream) {
  using namespace lt;
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || cp_rank < 0 || cp_rank >= cp_world) return -int(kStatusBadArgument);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (phase == 0)
    return bwd_delta(o, do_ptrs[cp_rank], const_cast<float*>(delta_ptrs[cp_rank]), B, Tq, Hq, D, so_b, so_t, sdo_b, sdo_t, st);
  if (phase == 1)
    return bwd_main(q_ptrs, k, v, do_ptrs, lse_ptrs, delta_ptrs, dq_acc_ptrs, dk, dv, B, Tq, Tk, Hq, Hkv, D, sq_b, sq_t, sk_b, sk_t,
                    sv_b, sv_t, sdo_b, sdo_t, sdk_b, sdk_t, scale, causal, cp_world, cp_rank, zigzag, st);
  return bwd_convert(dq_acc_ptrs[cp_rank], dq, B, Tq, Hq, D, sdq_b, sdq_t, st);
}

}  // extern "C"
