// ZeRO-3 / tensor-parallel fused communication kernels over NVLink peer memory.
//
// 1. lt_ag_gemm_bf16: all-gather fused into the consuming GEMM.  One operand (a weight sharded by rows over
//    the ranks for FSDP, or a sequence-sharded activation for tensor parallelism) lives as W row shards in
//    the ranks' symmetric memory.  A few "gather" CTAs of the SAME kernel pull the shards chunk by chunk
//    with bulk async copies (peer HBM -> shared memory -> local staging buffer; plain, non-multicast
//    copies), publish a flag per chunk, and the GEMM CTAs' TMA producer waits (bounded) on the flag of the
//    chunk a tile needs.  Tiles are rastered in arrival order starting with the local shard, so the math
//    of early tiles hides the transfer of later chunks; each byte crosses NVLink once.
//    Replaces the reference's pre-forward all-gather hooks (src/distributed/fsdp_wrapper.cpp:123-145) and
//    ColumnParallelLinear's all-gather (src/nn/parallel_linear.cpp:38-51).
// 2. lt_rs_adamw: gradient reduce-scatter fused with the sharded AdamW update.  Each rank signals that its
//    gradient bucket is complete, waits (bounded) for the same signal of every peer, then reads its slice
//    of every rank's gradient buffer straight from peer memory (or reduced in the switch through a
//    multimem address), accumulates in fp32, applies AdamW to its fp32 master / m / v shard and writes the
//    bf16 parameter shard that the next step's gathers read.  Replaces the reduce-scatter grad hook plus
//    ZeRO3Optimizer::step (src/distributed/fsdp_wrapper.cpp:81-96, src/optim/zero3_optimizer.cpp:11-105).
// 3. lt_embedding_fwd_sharded: embedding rows fetched from the owning rank.
// 4. lt_signal_barrier: all-ranks barrier on symmetric flags (bounded wait).
#include "lt_cuda.h"
#include "comm_common.cuh"
#include "gemm_sm100_2cta.cuh"

namespace lt {

constexpr int kMaxRanks = 8;

struct GatherArgs {
  const __nv_bfloat16* shard[kMaxRanks];  // shard[r]: rows [r*rows_per_rank, (r+1)*rows_per_rank) of the matrix
  __nv_bfloat16* full;                    // local staging buffer [rows_total, cols]
  uint32_t* flags;                        // one per chunk, value = epoch once the chunk has landed
  uint32_t epoch;
  int world, rank;
  int rows_total, rows_per_rank, cols;
  int chunk_rows, n_chunks, chunk_rot;    // chunk o of the schedule is chunk (o + chunk_rot) % n_chunks
  int gate_dim;                           // 0: N block, 1: K block, 2: M block
  int n_comm;                             // number of gather CTAs (blockIdx.x < n_comm)
};

// What the gather CTAs fetch once their own operand is complete: the gathered operand of the NEXT GEMM of the
// layer sequence, into that GEMM's staging buffer and flags.  They stop when this kernel's tiles are done
// (`progress` reaches `progress_target`), and the next kernel's gather CTAs skip the chunks that already landed.
struct PrefetchArgs {
  GatherArgs next;                        // next.n_chunks == 0: nothing to prefetch
  uint32_t* progress;                     // tile-warp completions of the running kernel (monotonic counter)
  uint32_t progress_target;
};

struct ProgressDone {
  uint32_t* progress;
  __device__ __forceinline__ void fence() const {}
  __device__ __forceinline__ void operator()(int, int) const {
    if (progress) red_add_release_gpu(progress, 1u);
  }
};

// One thread of a gather CTA runs the whole copy pipeline.
__device__ void gather_cta(const GatherArgs& g_own, const PrefetchArgs& pf, int* status) {
  const GatherArgs& g = g_own;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kGatherStages * kGatherStageBytes);
  const uint32_t bb = smem_u32(bars);
  __shared__ int abort_flag_s;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGatherStages; ++s) mbar_init(bb + 8u * s, 1);
    abort_flag_s = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  volatile int* abort_flag = &abort_flag_s;
  uint32_t use[kGatherStages];
  for (int s = 0; s < kGatherStages; ++s) use[s] = 0;

  const int n_own = g.n_chunks;
  const int n_all = n_own + pf.next.n_chunks;
  for (int oo = blockIdx.x; oo < n_all; oo += g.n_comm) {
    const bool own = oo < n_own;
    const GatherArgs& g = own ? g_own : pf.next;
    const int o = own ? oo : oo - n_own;
    const long long row_bytes = (long long)g.cols * 2;
    int max_rows = int(kGatherStageBytes / row_bytes);
    if (max_rows < 1) max_rows = 1;  // rows wider than a stage are split by columns below
    if (!own && ld_acquire_gpu(pf.progress) >= pf.progress_target) return;   // the GEMM is done: leave the rest
    int c = o + g.chunk_rot;
    if (c >= g.n_chunks) c -= g.n_chunks;
    if (ld_acquire_gpu(g.flags + c) == g.epoch) continue;                     // already landed (prefetched earlier)
    const int r0 = c * g.chunk_rows;
    const int r1 = min(r0 + g.chunk_rows, g.rows_total);
    // Segment walker: contiguous pieces that stay inside one owner and one stage.
    int row = r0;
    long long col_b = 0;  // byte offset inside the row when rows are wider than a stage
    int issued = 0, stored = 0;
    // ring of pending segments (destination + size), indexed by stage
    void* seg_dst[kGatherStages];
    uint32_t seg_bytes[kGatherStages];
    auto next_segment = [&](const void*& src, void*& dst, uint32_t& bytes) -> bool {
      if (row >= r1) return false;
      const int owner = min(row / g.rows_per_rank, g.world - 1);
      const int local_row = row - owner * g.rows_per_rank;
      if (row_bytes > kGatherStageBytes) {
        const long long left = row_bytes - col_b;
        bytes = uint32_t(left < kGatherStageBytes ? left : kGatherStageBytes);
        src = reinterpret_cast<const uint8_t*>(g.shard[owner]) + (long long)local_row * row_bytes + col_b;
        dst = reinterpret_cast<uint8_t*>(g.full) + (long long)row * row_bytes + col_b;
        col_b += bytes;
        if (col_b >= row_bytes) { col_b = 0; ++row; }
      } else {
        int end = min(r1, min((owner + 1) * g.rows_per_rank, row + max_rows));
        if (owner == g.world - 1) end = min(r1, row + max_rows);
        bytes = uint32_t((end - row) * row_bytes);
        src = reinterpret_cast<const uint8_t*>(g.shard[owner]) + (long long)local_row * row_bytes;
        dst = reinterpret_cast<uint8_t*>(g.full) + (long long)row * row_bytes;
        row = end;
      }
      return true;
    };
    bool ok = true;
    bool more = true;
    while (ok && (more || stored < issued)) {
      // keep the ring full
      while (more && issued - stored < kGatherStages) {
        const void* src; void* dst; uint32_t bytes;
        if (!next_segment(src, dst, bytes)) { more = false; break; }
        const int s = issued % kGatherStages;
        // the stage's previous store must have finished reading shared memory
        tma_store_wait_read<0>();
        mbar_expect_tx(bb + 8u * s, bytes);
        bulk_g2s(sbase + s * kGatherStageBytes, src, bytes, bb + 8u * s);
        seg_dst[s] = dst;
        seg_bytes[s] = bytes;
        ++issued;
      }
      if (stored < issued) {
        const int s = stored % kGatherStages;
        if (!mbar_wait(bb + 8u * s, use[s] & 1u, abort_flag, status, kStatusTimeoutFull)) { ok = false; break; }
        use[s]++;
        bulk_s2g(seg_dst[s], sbase + s * kGatherStageBytes, seg_bytes[s]);
        tma_store_commit();
        ++stored;
      }
    }
    if (!ok) return;
    tma_store_wait<0>();
    asm volatile("fence.proxy.async.global;" ::: "memory");
    __threadfence();
    st_release_gpu(g.flags + c, g.epoch);
  }
}

template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
               const GatherArgs g, const PrefetchArgs pf) {
  if (int(blockIdx.x) < g.n_comm) {
    gather_cta(g, pf, p.status);
    return;
  }
  // GEMM CTAs see a grid that starts at n_comm.
  FlagGate gate{g.flags, g.epoch, g.gate_dim, -1};
  gemm_body<BLOCK_N, A_MAJOR, B_MAJOR>(&tmA, &tmB, p, gate, ProgressDone{pf.progress}, g.n_comm);
}

// The same kernel on CTA pairs (256 x 256 tiles, cta_group::2).  n_comm is even, so gather CTAs pair with gather CTAs
// and never take part in a pair's barriers.
template <int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                    const GatherArgs g, const PrefetchArgs pf) {
  if (int(blockIdx.x) < g.n_comm) {
    gather_cta(g, pf, p.status);
    return;
  }
  FlagGate gate{g.flags, g.epoch, g.gate_dim, -1};
  gemm_body_pair<A_MAJOR, B_MAJOR>(&tmA, &tmB, p, gate, ProgressDone{pf.progress}, g.n_comm);
}

// ---------------------------------------------------------------------------------------------- RS + AdamW
struct RsSeg {
  long long full_off;   // element offset of this rank's rows inside the full gradient buffer
  long long shard_off;  // element offset inside the rank's shard buffers
  long long n;          // elements (multiple of 8)
};
struct RsAdamArgs {
  const __nv_bfloat16* grads[kMaxRanks];  // every rank's full gradient buffer (peer pointers)
  const __nv_bfloat16* mc_grads;          // multimem address of the same buffer, or nullptr
  float* master;
  float* m;
  float* v;
  __nv_bfloat16* param_shard;
  RsSeg seg[8];
  int n_seg;
  float lr, beta1, beta2, eps, wd, bc1, bc2;
  uint32_t* my_flags;                 // local signal words [slots][kMaxRanks]
  uint32_t* peer_flags[kMaxRanks];    // the same array on every rank
  int slot;
  uint32_t epoch;
  int world, rank;
  int* status;
};

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], uint4 u) {
  float2 f;
  f = unpack_bf16x2(u.x); acc[0] += f.x; acc[1] += f.y;
  f = unpack_bf16x2(u.y); acc[2] += f.x; acc[3] += f.y;
  f = unpack_bf16x2(u.z); acc[4] += f.x; acc[5] += f.y;
  f = unpack_bf16x2(u.w); acc[6] += f.x; acc[7] += f.y;
}

// 128 threads per CTA: with ~120 registers a CTA then takes under a quarter of an SM's register file, so it can run
// on an SM that a persistent GEMM CTA (192 threads x 200-232 registers) already occupies; a 256-thread CTA cannot,
// and the whole kernel would wait for the gaps between GEMMs instead of running beside them.
constexpr int kRsAdamThreads = 128;
__global__ void __launch_bounds__(kRsAdamThreads) rs_adamw_kernel(const RsAdamArgs a) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  // 1. tell every peer that this rank's gradients for the bucket are complete, then wait for all of them
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.peer_flags[threadIdx.x] + a.slot * kMaxRanks + a.rank, a.epoch);
  }
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge_sys(a.my_flags + a.slot * kMaxRanks + threadIdx.x, a.epoch, a.status)) ok_s = 0;
  }
  __syncthreads();
  if (!ok_s) return;
  // 2. reduce my slice over the ranks and update
  for (int s = 0; s < a.n_seg; ++s) {
    const RsSeg sg = a.seg[s];
    const long long n8 = sg.n / 8;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const long long fo = sg.full_off + i * 8;
      const long long so = sg.shard_off + i * 8;
      // every load of the iteration is issued before the first use: the optimizer state (HBM) travels under the
      // NVLink latency of the peers' gradients instead of after it
      uint4 u[kMaxRanks];
      if (a.mc_grads) {
        u[0] = multimem_ld_reduce_bf16x8(a.mc_grads + fo);
      } else {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < a.world) u[r] = ld_relaxed_sys_v4(a.grads[r] + fo);
      }
      float4 p0 = __ldcs(reinterpret_cast<const float4*>(a.master + so)), p1 = __ldcs(reinterpret_cast<const float4*>(a.master + so + 4));
      float4 m0 = __ldcs(reinterpret_cast<const float4*>(a.m + so)), m1 = __ldcs(reinterpret_cast<const float4*>(a.m + so + 4));
      float4 v0 = __ldcs(reinterpret_cast<const float4*>(a.v + so)), v1 = __ldcs(reinterpret_cast<const float4*>(a.v + so + 4));
      if (a.mc_grads) {
        acc_bf16x8(g, u[0]);
      } else {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < a.world) acc_bf16x8(g, u[r]);
      }
      float pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * g[j];
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * g[j] * g[j];
        float p = pp[j];
        p -= a.lr * a.wd * p;
        p -= a.lr * (mm[j] / a.bc1) / (sqrtf(vv[j] / a.bc2) + a.eps);
        pp[j] = p;
      }
      *reinterpret_cast<float4*>(a.master + so) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(a.master + so + 4) = make_float4(pp[4], pp[5], pp[6], pp[7]);
      *reinterpret_cast<float4*>(a.m + so) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(a.m + so + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(a.v + so) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(a.v + so + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
      uint4 o;
      o.x = pack_bf16x2(pp[0], pp[1]); o.y = pack_bf16x2(pp[2], pp[3]);
      o.z = pack_bf16x2(pp[4], pp[5]); o.w = pack_bf16x2(pp[6], pp[7]);
      *reinterpret_cast<uint4*>(a.param_shard + so) = o;
    }
  }
}

// ---------------------------------------------------------------------------------------------- misc
struct PeerPtrs {
  const __nv_bfloat16* p[kMaxRanks];
};
__global__ void embedding_fwd_sharded_kernel(const long long* __restrict__ idx, PeerPtrs tables, __nv_bfloat16* __restrict__ out,
                                             long long n_tok, int D, int V, int rows_per_rank, int world) {
  const int vpr = D / 8;
  const long long total = n_tok * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = int(i % vpr) * 8;
    long long t = idx[r];
    t = t < 0 ? 0 : (t >= V ? V - 1 : t);
    int owner = int(t / rows_per_rank);
    if (owner >= world) owner = world - 1;
    const long long local = t - (long long)owner * rows_per_rank;
    *reinterpret_cast<uint4*>(out + r * D + c) = ld_relaxed_sys_v4(tables.p[owner] + local * D + c);
  }
}

struct BarrierArgs {
  uint32_t* my_flags;
  uint32_t* peer_flags[kMaxRanks];
  int slot;
  uint32_t epoch;
  int world, rank;
  int* status;
};
__global__ void signal_barrier_kernel(const BarrierArgs a) {
  if (threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.peer_flags[threadIdx.x] + a.slot * kMaxRanks + a.rank, a.epoch);
    wait_flag_ge_sys(a.my_flags + a.slot * kMaxRanks + threadIdx.x, a.epoch, a.status);
  }
}


// ---------------------------------------------------------------------------------------------- shard gather
// Weight all-gather without a GEMM attached: pulls `world` row shards of up to 8 matrices from the ranks'
// parameter buffers into local full-size staging areas with 16-byte peer loads, four in flight per thread.
// Used one layer ahead on a side stream when the GEMM's own gather slot is taken by the tensor-parallel
// activation gather (FSDP x TP): the next layer's weights need a fraction of the link rate, so a few CTAs
// that share SMs with the running GEMM are enough.  Same role as the reference's pre-forward all-gather
// (src/distributed/fsdp_wrapper.cpp:123-145), read from peer memory instead of through NCCL.
struct ShardGatherArgs {
  const __nv_bfloat16* shard[kMaxRanks];   // every rank's parameter shard buffer (peer-mapped)
  __nv_bfloat16* dst[8];                   // staging area of segment s (holds world * n elements)
  long long shard_off[8], n[8];            // element offset in the shard buffer, elements per rank
  long long vec_end[8];                    // running total of 16-byte vectors up to and including segment s
  int n_seg, world;
};
// 128-thread CTAs of < 48 registers: three of them fit beside a persistent GEMM CTA on the same SM.
constexpr int kShardGatherThreads = 128;
__global__ void __launch_bounds__(kShardGatherThreads) shard_gather_kernel(const ShardGatherArgs a) {
  const long long total = a.vec_end[a.n_seg - 1];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long base = blockIdx.x * (long long)blockDim.x + threadIdx.x; base < total; base += 4 * stride) {
    uint4 v[4];
    __nv_bfloat16* out[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long i = base + u * stride;
      out[u] = nullptr;
      if (i >= total) continue;
      int s = 0;
      while (i >= a.vec_end[s]) ++s;
      const long long j = i - (s ? a.vec_end[s - 1] : 0);      // vector index inside segment s
      const long long per_rank = a.n[s] / 8;
      const int r = int(j / per_rank);
      const long long e = (j - r * per_rank) * 8;
      v[u] = ld_relaxed_sys_v4(a.shard[r] + a.shard_off[s] + e);
      out[u] = a.dst[s] + r * a.n[s] + e;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (out[u]) *reinterpret_cast<uint4*>(out[u]) = v[u];
  }
}


template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
static int launch_ag_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const GatherArgs& g,
                          const PrefetchArgs& pf, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool configured = false;
  auto kern = ag_gemm_kernel<BLOCK_N, A_MAJOR, B_MAJOR>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(tmA, tmB, p, g, pf);
  LT_LAUNCH_CHECK();
  return 0;
}

template <int A_MAJOR, int B_MAJOR>
static int launch_ag_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const GatherArgs& g,
                               const PrefetchArgs& pf, int grid, cudaStream_t st) {
  static bool configured = false;
  auto kern = ag_gemm_pair_kernel<A_MAJOR, B_MAJOR>;
  constexpr int kSmem = kPairSmemBytes > kGatherStages * kGatherStageBytes + 2048 ? kPairSmemBytes
                                                                                  : kGatherStages * kGatherStageBytes + 2048;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    configured = true;
  }
  kern<<<grid, kGemmThreads, kSmem, st>>>(tmA, tmB, p, g, pf);
  LT_LAUNCH_CHECK();
  return 0;
}

// Whether a gather-GEMM of this shape runs on CTA pairs (the decision must be the same wherever tile counts are
// derived: the kernel launch, the progress target of a prefetch and lt_gemm_num_tiles).
// Gather CTAs for one call when the caller leaves the choice open.  One gather CTA moves 20-30 GB/s (its bulk copies are
// bound by the requests a single SM keeps in flight over NVLink) but whole chunks land late, so the model counts
// 14 GB/s; the gather's rate grows with the CTAs given to it while the GEMM loses those SMs.  Picks the count (a
// multiple of 4, so that CTA pairs stay aligned) with the smallest larger-of-the-two time, never fewer than 8.
// Measured on [8192, 3584, 4096] with half of A remote: 8 / 12 / 16 / 24 gather CTAs take 0.295 / 0.265 / 0.242 /
// 0.270 ms.
static int pick_gather_ctas(double flops, double remote_bytes, int sms) {
  constexpr double kPerCtaBytesPerSec = 14e9;
  constexpr double kPerSmFlopsPerSec = 1.5e15 / 148.0;
  int best = 8;
  double best_t = 1e30;
  for (int n = 8; n <= 32 && n <= sms / 2; n += 4) {
    const double t_gemm = flops / (kPerSmFlopsPerSec * (sms - n));
    const double t_gather = remote_bytes / (kPerCtaBytesPerSec * n);
    const double t = t_gemm > t_gather ? t_gemm : t_gather;
    if (t < best_t * 0.999) { best_t = t; best = n; }
  }
  return best;
}

static bool ag_use_pairs(int M, int n_comm, int sms) {
  return gemm_pair_mode() > 0 && M > kBlockM && (n_comm % 2 == 0) && ((sms - n_comm) % 2 == 0);
}

}  // namespace lt

namespace lt {
// Chunking of a gathered operand for a GEMM of shape (M, N, K) with tile width block_n.
static void setup_gather(GatherArgs& g, int gather_operand, int M, int N, int K, int block_n, int rank, int rows_per_rank,
                         int& rot_out) {
  const int m_blocks = (M + kBlockM - 1) / kBlockM, n_blocks = (N + block_n - 1) / block_n, k_blocks = (K + kBlockK - 1) / kBlockK;
  const int first_row = rank * rows_per_rank;
  if (gather_operand == 0) {
    g.rows_total = M; g.cols = K; g.chunk_rows = kBlockM; g.gate_dim = 2; g.n_chunks = m_blocks;
  } else if (gather_operand == 1) {
    g.rows_total = N; g.cols = K; g.chunk_rows = block_n; g.gate_dim = 0; g.n_chunks = n_blocks;
  } else {
    g.rows_total = K; g.cols = N; g.chunk_rows = kBlockK; g.gate_dim = 1; g.n_chunks = k_blocks;
  }
  g.chunk_rot = (first_row / g.chunk_rows) % g.n_chunks;
  rot_out = g.chunk_rot;
}
}  // namespace lt

extern "C" {

// LtNextGather (lt_cuda.h): description of the next gather-GEMM of the sequence, for prefetching.

// GEMM whose gathered operand is assembled from `world` row shards while the kernel runs.
//   gather_operand: 0 = A (stored [M, K], rows sharded, tiles gated by M block),
//                   1 = B stored [N, K] (b_major 0, gated by N block),
//                   2 = B stored [K, N] (b_major 1, rows = reduction dim, gated by K block).
//   shard_ptrs[r]: rank r's shard (rows_per_rank x cols, contiguous), a peer-mapped pointer.
//   full: local staging buffer [rows_total, cols] the TMA descriptor of that operand reads.
//   flags: device array with one word per chunk (>= 4096 entries); epoch must grow with every call that
//   reuses the flags.  n_comm: gather CTAs (0 = chosen from the GEMM's FLOPs and the bytes to fetch).
int lt_ag_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                    int a_major, int b_major, int out_fp32, const void* bias, const void* residual, long long ldr, int act,
                    int accumulate, float alpha, int gather_operand, const void* const* shard_ptrs, int world, int rank,
                    int rows_per_rank, void* full, void* flags, unsigned epoch, int n_comm, const LtNextGather* next,
                    void* progress, unsigned progress_base, void* stream) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > kMaxRanks) return -int(kStatusBadArgument);
  if ((gather_operand == 0 && a_major != 0) || (gather_operand == 1 && b_major != 0) || (gather_operand == 2 && b_major != 1))
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  if (n_comm <= 0) {
    const double rows = gather_operand == 0 ? double(M) : double(N);
    n_comm = pick_gather_ctas(2.0 * M * N * K, double(world - 1) / world * rows * K * 2.0, sms);
  }
  if (n_comm > sms / 2) n_comm = sms / 2;
  const bool pairs = ag_use_pairs(M, n_comm, sms);
  int block_n = pairs ? kPairBlockN : pick_block_n(M, N, sms - n_comm);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.act = act; p.accumulate = accumulate; p.alpha = alpha;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  GatherArgs g{};
  for (int r = 0; r < world; ++r) g.shard[r] = static_cast<const __nv_bfloat16*>(shard_ptrs[r]);
  g.full = static_cast<__nv_bfloat16*>(full);
  g.flags = static_cast<uint32_t*>(flags);
  g.epoch = epoch;
  g.world = world; g.rank = rank;
  g.rows_per_rank = rows_per_rank;
  g.n_comm = n_comm;
  int rot = 0;
  setup_gather(g, gather_operand, M, N, K, block_n, rank, rows_per_rank, rot);
  if (pairs) fill_pair_tiles(p);
  if (gather_operand == 0) {
    // A arrives by 128-row chunks starting at this rank's rows.  All N blocks of one M block before the next M block
    // would stream the whole B operand from DRAM once per M block; instead M blocks are taken in groups (B tiles are
    // reused across the group out of L2) and the groups start at the one that holds the local rows.
    const int m_rot = pairs ? rot / 2 : rot;   // chunks of A are 128 rows, pair tiles 256
    if (p.m_blocks % p.group_m == 0 && p.m_blocks > p.group_m) { p.raster = 0; p.rot = m_rot / p.group_m; }
    else { p.raster = 2; p.rot = m_rot; }
  }
  else if (gather_operand == 1) { p.raster = 1; p.rot = rot; }
  else { p.k_rot = rot; }
  PrefetchArgs pf{};
  pf.progress = static_cast<uint32_t*>(progress);
  pf.progress_target = progress_base + uint32_t(p.num_tiles) * (pairs ? 8u : 4u);   // epilogue warps per tile
  if (next && progress && next->M > 0) {
    GatherArgs& n = pf.next;
    for (int r = 0; r < world; ++r) n.shard[r] = static_cast<const __nv_bfloat16*>(next->shard_ptrs[r]);
    n.full = static_cast<__nv_bfloat16*>(next->full);
    n.flags = static_cast<uint32_t*>(next->flags);
    n.epoch = next->epoch;
    n.world = world; n.rank = rank; n.rows_per_rank = next->rows_per_rank; n.n_comm = n_comm;
    int nrot = 0;
    setup_gather(n, next->gather_operand, next->M, next->N, next->K,
                 ag_use_pairs(next->M, n_comm, sms) ? kPairBlockN : pick_block_n(next->M, next->N, sms - n_comm), rank,
                 next->rows_per_rank, nrot);
    if ((long long)n.cols * 2 % 16 != 0) n.n_chunks = 0;
  }
  if ((long long)g.cols * 2 % 16 != 0) return -int(kStatusBadArgument);
  CUtensorMap tmA, tmB;
  int r = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_major, b_major, pairs ? kPairBlockN / 2 : block_n);
  if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pairs) {
    int grid = sms;
    if ((grid - n_comm) / 2 > p.num_tiles) grid = 2 * p.num_tiles + n_comm;
    if (a_major != 0) return -int(kStatusBadArgument);
    return b_major ? launch_ag_gemm_pair<0, 1>(tmA, tmB, p, g, pf, grid, st) : launch_ag_gemm_pair<0, 0>(tmA, tmB, p, g, pf, grid, st);
  }
  int grid = sms;
  if (grid - n_comm > p.num_tiles) grid = p.num_tiles + n_comm;
  const int key = (block_n == 256 ? 4 : 0) | (a_major ? 2 : 0) | (b_major ? 1 : 0);
  switch (key) {
    case 0: return launch_ag_gemm<128, 0, 0>(tmA, tmB, p, g, pf, grid, st);
    case 1: return launch_ag_gemm<128, 0, 1>(tmA, tmB, p, g, pf, grid, st);
    case 4: return launch_ag_gemm<256, 0, 0>(tmA, tmB, p, g, pf, grid, st);
    case 5: return launch_ag_gemm<256, 0, 1>(tmA, tmB, p, g, pf, grid, st);
    default: return -int(kStatusBadArgument);
  }
}

// Tile count of a gather-GEMM in units of four epilogue-warp completions (what the progress counter advances by).
int lt_gemm_num_tiles(int M, int N, int n_comm) {
  using namespace lt;
  if (n_comm <= 0) n_comm = 8;
  if (ag_use_pairs(M, n_comm, sm_count()))
    return 2 * ((M + kPairBlockM - 1) / kPairBlockM) * ((N + kPairBlockN - 1) / kPairBlockN);
  const int bn = pick_block_n(M, N, sm_count() - n_comm);
  return ((M + kBlockM - 1) / kBlockM) * ((N + bn - 1) / bn);
}

// segs: n_seg triples (full_off, shard_off, n) in elements, n a multiple of 8.
int lt_rs_adamw(const void* const* grad_ptrs, const void* mc_grads, float* master, float* m, float* v, void* param_shard,
                const long long* segs, int n_seg, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                float bc2, void* my_flags, const void* const* peer_flags, int slot, unsigned epoch, int world, int rank,
                int max_ctas, void* stream) {
  using namespace lt;
  if (world < 1 || world > kMaxRanks || n_seg < 0 || n_seg > 8) return -int(kStatusBadArgument);
  RsAdamArgs a{};
  for (int r = 0; r < world; ++r) {
    a.grads[r] = static_cast<const __nv_bfloat16*>(grad_ptrs[r]);
    a.peer_flags[r] = static_cast<uint32_t*>(const_cast<void*>(peer_flags[r]));
  }
  a.mc_grads = static_cast<const __nv_bfloat16*>(mc_grads);
  a.master = master; a.m = m; a.v = v;
  a.param_shard = static_cast<__nv_bfloat16*>(param_shard);
  long long total = 0;
  for (int s = 0; s < n_seg; ++s) {
    a.seg[s].full_off = segs[3 * s]; a.seg[s].shard_off = segs[3 * s + 1]; a.seg[s].n = segs[3 * s + 2];
    if (a.seg[s].n % 8 != 0 || a.seg[s].full_off % 8 != 0 || a.seg[s].shard_off % 8 != 0) return -int(kStatusBadArgument);
    total += a.seg[s].n;
  }
  a.n_seg = n_seg;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.bc1 = bc1; a.bc2 = bc2;
  a.my_flags = static_cast<uint32_t*>(my_flags);
  a.slot = slot; a.epoch = epoch; a.world = world; a.rank = rank;
  a.status = device_status_word();
  long long blocks = (total / 8 + kRsAdamThreads - 1) / kRsAdamThreads;
  long long cap = max_ctas > 0 ? max_ctas : (long long)sm_count() * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  rs_adamw_kernel<<<(unsigned)blocks, kRsAdamThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LT_LAUNCH_CHECK();
  return 0;
}

// Copies, for each of n_seg segments, `n` elements starting at `shard_off` of every rank's shard buffer into
// dst[s] + r * n (rank order).  segs: n_seg triples (shard_off, n, unused) in elements, multiples of 8;
// dst_ptrs: n_seg local destination pointers, 16-byte aligned.  max_ctas: 0 = 64 (of 128 threads).
int lt_gather_shards(const void* const* shard_ptrs, int world, const long long* segs, const void* const* dst_ptrs, int n_seg,
                     int max_ctas, void* stream) {
  using namespace lt;
  if (world < 1 || world > kMaxRanks || n_seg < 1 || n_seg > 8) return -int(kStatusBadArgument);
  ShardGatherArgs a{};
  for (int r = 0; r < world; ++r) a.shard[r] = static_cast<const __nv_bfloat16*>(shard_ptrs[r]);
  long long total = 0;
  for (int s = 0; s < n_seg; ++s) {
    a.shard_off[s] = segs[3 * s]; a.n[s] = segs[3 * s + 1];
    a.dst[s] = static_cast<__nv_bfloat16*>(const_cast<void*>(dst_ptrs[s]));
    if (a.n[s] <= 0 || a.n[s] % 8 != 0 || a.shard_off[s] % 8 != 0 || (reinterpret_cast<uintptr_t>(a.dst[s]) & 15) != 0)
      return -int(kStatusBadArgument);
    total += a.n[s] / 8 * world;
    a.vec_end[s] = total;
  }
  a.n_seg = n_seg; a.world = world;
  long long blocks = (total + 4 * kShardGatherThreads - 1) / (4 * kShardGatherThreads);
  const long long cap = max_ctas > 0 ? max_ctas : 64;
  if (blocks > cap) blocks = cap;
  shard_gather_kernel<<<(unsigned)blocks, kShardGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_embedding_fwd_sharded(const long long* idx, const void* const* table_ptrs, void* out, long long n_tok, int D, int V,
                             int rows_per_rank, int world, void* stream) {
  using namespace lt;
  if (D % 8 != 0 || world < 1 || world > kMaxRanks) return -int(kStatusBadArgument);
  if (n_tok == 0) return 0;
  PeerPtrs t{};
  for (int r = 0; r < world; ++r) t.p[r] = static_cast<const __nv_bfloat16*>(table_ptrs[r]);
  long long blocks = (n_tok * (D / 8) + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  embedding_fwd_sharded_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      idx, t, static_cast<__nv_bfloat16*>(out), n_tok, D, V, rows_per_rank, world);
  LT_LAUNCH_CHECK();
  return 0;
}

int lt_signal_barrier(void* my_flags, const void* const* peer_flags, int slot, unsigned epoch, int world, int rank, void* stream) {
  using namespace lt;
  if (world < 1 || world > kMaxRanks) return -int(kStatusBadArgument);
  BarrierArgs a{};
  a.my_flags = static_cast<uint32_t*>(my_flags);
  for (int r = 0; r < world; ++r) a.peer_flags[r] = static_cast<uint32_t*>(const_cast<void*>(peer_flags[r]));
  a.slot = slot; a.epoch = epoch; a.world = world; a.rank = rank;
  a.status = device_status_word();
  signal_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
