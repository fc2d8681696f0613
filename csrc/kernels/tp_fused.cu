// GEMM fused with the reduce-scatter that follows it (RowParallelLinear / o-proj / down-proj under sequence
// parallelism, and the input gradient of ColumnParallelLinear).
//
// Every rank multiplies its K-slice: partial[M, N] = A[M, K_local] * op(B).  Rank r owns rows
// [r*M/W, (r+1)*M/W) of the result.  Instead of writing the partial product locally and calling a
// reduce-scatter afterwards (the reference all-reduces after the GEMM: src/nn/parallel_linear.cpp:87-106),
// the epilogue of each tcgen05 tile stores its rows straight into the owner's staging buffer over NVLink
// (plain peer stores), then bumps a per-row-block arrival counter on the owner with a system-scope release.
// Tiles are computed for the other ranks first and for this rank last, so the transfers overlap the math.
// When its own tiles are done, the same kernel sums the W staged partials of every local row block as soon as
// the block's counter shows that all ranks delivered it (bounded wait) and writes the bf16 result, optionally
// adding a bias and a residual.
#include "lt_cuda.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"

namespace lt {

constexpr int kRsMaxRanks = 8;

struct RsArgs {
  const __nv_bfloat16* stage;        // local staging buffer [W][rows_per_rank][N] (what the peers wrote)
  uint32_t* my_counters;             // [rows_per_rank / 128] arrival counters on this rank
  uint32_t* peer_counters[kRsMaxRanks];
  uint32_t target;                   // counter value once every rank delivered every tile of a row block
  __nv_bfloat16* out;                // [rows_per_rank, N]
  long long ldo;
  const __nv_bfloat16* bias;         // [N] or nullptr
  const __nv_bfloat16* residual;     // [rows_per_rank, N] or nullptr
  long long ldr;
  int world, rank, rows_per_rank, N, block_n;
};

struct ArriveDone {
  uint32_t* const* peer_counters;
  int rows_per_rank;
  int total_rows;
  int rank;
  // No fence per lane: the lanes' stores are ordered before lane 0's release by the warp barrier between them, and a
  // release is cumulative.  A system-scope fence in every lane of every tile cost more than the tile's main loop.
  __device__ __forceinline__ void fence() const {}
  __device__ __forceinline__ void operator()(int m_blk, int) const {
    const int row0 = m_blk * kBlockM;
    if (row0 >= total_rows) return;   // the odd CTA of a pair past the last row block
    const int owner = row0 / rows_per_rank;
    const int local_blk = (row0 - owner * rows_per_rank) / kBlockM;
    if (owner == rank) red_add_release_gpu(peer_counters[owner] + local_blk, 1u);   // own rows: nothing left this GPU
    else red_add_release_sys(peer_counters[owner] + local_blk, 1u);
  }
};

// Second phase of the fused kernels: sum the W staged partials of every local row block once its arrival counter
// shows that all ranks delivered it (bounded wait), add bias / residual, write bf16.
__device__ __forceinline__ void rs_reduce_phase(const GemmParams& p, const RsArgs& a) {
  // Work items are (local 128-row block, 256-column slice) pairs spread over every CTA of the grid, and a thread keeps
  // the loads of several 16-byte vectors of all W partials in flight: with one CTA per row block and one vector per
  // thread this phase, not the GEMM, set the kernel's duration.
  __shared__ int ok_s;
  constexpr int kSlice = 256;
  constexpr int kVecPerRow = kSlice / 8;
  constexpr int kUnroll = 4;
  const int local_blocks = a.rows_per_rank / kBlockM;
  const int col_slices = (a.N + kSlice - 1) / kSlice;
  const long long slot = (long long)a.rows_per_rank * a.N;
  int last_lb = -1;
  for (int item = blockIdx.x; item < local_blocks * col_slices; item += gridDim.x) {
    const int lb = item / col_slices, cs = item % col_slices;
    if (lb != last_lb) {
      if (threadIdx.x == 0) ok_s = wait_flag_ge_sys(a.my_counters + lb, a.target, p.status) ? 1 : 0;
      __syncthreads();
      const int ok = ok_s;
      __syncthreads();
      if (!ok) return;
      last_lb = lb;
    }
    const int total = kBlockM * kVecPerRow;
    for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * kUnroll) {
      uint4 u[kUnroll][kRsMaxRanks];
      int rr[kUnroll], cc[kUnroll];
      bool on[kUnroll];
#pragma unroll
      for (int q = 0; q < kUnroll; ++q) {
        const int i = i0 + q * blockDim.x;
        rr[q] = lb * kBlockM + i / kVecPerRow;
        cc[q] = cs * kSlice + (i % kVecPerRow) * 8;
        on[q] = (i < total) && (cc[q] < a.N);
        if (on[q]) {
#pragma unroll
          for (int src = 0; src < kRsMaxRanks; ++src)
            if (src < a.world) u[q][src] = ld_relaxed_sys_v4(a.stage + src * slot + (long long)rr[q] * a.N + cc[q]);
        }
      }
#pragma unroll
      for (int q = 0; q < kUnroll; ++q) {
        if (!on[q]) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        auto add8 = [&](const uint4& v) {
          float2 f;
          f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
          f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
          f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
          f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
        };
#pragma unroll
        for (int src = 0; src < kRsMaxRanks; ++src)
          if (src < a.world) add8(u[q][src]);
        if (a.bias) add8(*reinterpret_cast<const uint4*>(a.bias + cc[q]));
        if (a.residual) add8(*reinterpret_cast<const uint4*>(a.residual + (long long)rr[q] * a.ldr + cc[q]));
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(a.out + (long long)rr[q] * a.ldo + cc[q]) = o;
      }
    }
  }
}

template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
               const RsArgs a) {
  ArriveDone done{a.peer_counters, a.rows_per_rank, p.M, a.rank};
  gemm_body<BLOCK_N, A_MAJOR, B_MAJOR>(&tmA, &tmB, p, NoGate(), done);
  rs_reduce_phase(p, a);
}

template <int BLOCK_N, int A_MAJOR, int B_MAJOR>
static int launch_gemm_rs(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const RsArgs& a, int grid,
                          cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool configured = false;
  auto kern = gemm_rs_kernel<BLOCK_N, A_MAJOR, B_MAJOR>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(tmA, tmB, p, a);
  LT_LAUNCH_CHECK();
  return 0;
}

template <int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_rs_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                    const RsArgs a, const __grid_constant__ ScatterMaps sm) {
  ArriveDone done{a.peer_counters, a.rows_per_rank, p.M, a.rank};
  gemm_body_pair<A_MAJOR, B_MAJOR>(&tmA, &tmB, p, NoGate(), done, 0, &sm);
  rs_reduce_phase(p, a);
}

template <int A_MAJOR, int B_MAJOR>
static int launch_gemm_rs_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, const RsArgs& a,
                               const ScatterMaps& sm, int grid, cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_rs_pair_kernel<A_MAJOR, B_MAJOR>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairScatterSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, kPairScatterSmemBytes, st>>>(tmA, tmB, p, a, sm);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // namespace lt

extern "C" {

// out[rows_per_rank, N] = sum over ranks of (A_r[M, K] * op(B_r))[rank's rows] (+ bias + residual).
//   stage_ptrs[r]: rank r's staging buffer [world][rows_per_rank][N] bf16 (peer-mapped);
//   counter_ptrs[r]: rank r's arrival counters (one uint32 per local 128-row block), monotonic: `epoch` is the
//   number of calls made so far on these counters, including this one.
//   M must equal world * rows_per_rank, rows_per_rank a multiple of 128, N a multiple of 8.
int lt_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int b_major,
                    const void* const* stage_ptrs, const void* const* counter_ptrs, unsigned epoch, int world, int rank,
                    int rows_per_rank, void* out, long long ldo, const void* bias, const void* residual, long long ldr,
                    void* stream) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > kRsMaxRanks || rows_per_rank % kBlockM != 0 || M != world * rows_per_rank || N % 8 != 0)
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  const bool pairs = gemm_pair_mode() > 0 && M > kBlockM && sms % 2 == 0;
  const int block_n = pairs ? kPairBlockN : pick_block_n(M, N, sms);
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = nullptr; p.ldc = N; p.out_fp32 = 0;
  p.alpha = 1.f;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  for (int r = 0; r < world; ++r) p.peer_C[r] = const_cast<void*>(stage_ptrs[r]);
  p.rows_per_rank = rows_per_rank;
  p.src_rank = rank;
  // rows of the other ranks first (starting with rank + 1), this rank's rows last
  if (pairs) fill_pair_tiles(p);
  p.raster = 2;
  p.rot = (((rank + 1) % world) * rows_per_rank) / (pairs ? kPairBlockM : kBlockM);
  RsArgs a{};
  a.stage = static_cast<const __nv_bfloat16*>(stage_ptrs[rank]);
  a.my_counters = static_cast<uint32_t*>(const_cast<void*>(counter_ptrs[rank]));
  for (int r = 0; r < world; ++r) a.peer_counters[r] = static_cast<uint32_t*>(const_cast<void*>(counter_ptrs[r]));
  a.target = epoch * uint32_t(world) * uint32_t(p.n_blocks) * 4u;  // 4 epilogue warps signal per tile
  a.out = static_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr;
  a.world = world; a.rank = rank; a.rows_per_rank = rows_per_rank; a.N = N; a.block_n = block_n;
  CUtensorMap tmA, tmB;
  int r = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, 0, b_major, pairs ? kPairBlockN / 2 : block_n);
  if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pairs) {
    const int grid2 = 2 * (sms / 2 < p.num_tiles ? sms / 2 : p.num_tiles);
    ScatterMaps sm;
    for (int q = 0; q < kRsMaxRanks; ++q) {
      const void* base = stage_ptrs[q < world ? q : 0];
      const int e = encode_tmap_2d(&sm.m[q], base, 2, (uint64_t)N, (uint64_t)M, (uint64_t)N * 2, 64, 32, 1);
      if (e) return 3000 + e;
    }
    return b_major ? launch_gemm_rs_pair<0, 1>(tmA, tmB, p, a, sm, grid2, st)
                   : launch_gemm_rs_pair<0, 0>(tmA, tmB, p, a, sm, grid2, st);
  }
  int grid = sms < p.num_tiles ? sms : p.num_tiles;
  if (block_n == 256) return b_major ? launch_gemm_rs<256, 0, 1>(tmA, tmB, p, a, grid, st) : launch_gemm_rs<256, 0, 0>(tmA, tmB, p, a, grid, st);
  return b_major ? launch_gemm_rs<128, 0, 1>(tmA, tmB, p, a, grid, st) : launch_gemm_rs<128, 0, 0>(tmA, tmB, p, a, grid, st);
}

}  // extern "C"
