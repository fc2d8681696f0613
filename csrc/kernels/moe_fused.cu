// Mixture-of-experts dispatch and combine fused with the grouped expert GEMMs (expert parallelism).
//
// The reference MoE is single-process, launches every expert over all tokens with one thread per token
// (src/nn/moe.cpp:167-261, src/backend/gpu_native/nn/nn_kernels.cu:1424-1493) and has no all-to-all.  Here the
// tokens never travel through a separate collective:
//
//  * lt_moe_gather_gemm  (dispatch -> grouped GEMM): the rows routed to this rank's experts are listed in a slot
//    table (source rank, source row), grouped by expert in blocks of 128 slots.  Gather CTAs of the GEMM kernel pull
//    those rows out of the source ranks' token buffers (plain bulk copies, peer HBM -> shared memory -> local slot
//    buffer) block by block and publish a flag per 128-slot block; the tcgen05 tiles of a block start as soon as its
//    flag is up and use the weight of the block's expert (B rows offset by expert).  The all-to-all "dispatch" is the
//    operand fetch of the GEMM.
//  * lt_moe_gemm_scatter (grouped GEMM -> combine): the epilogue multiplies every slot's row by its gate weight and
//    adds it straight into the fp32 output accumulator of the rank that owns the token (`red.add` to peer memory),
//    so the all-to-all "combine" and the weighted sum over the k experts are the GEMM epilogue.
// The same two kernels serve the backward pass with the roles swapped (gather dY rows for dH; scatter dX rows).
#include "lt_cuda.h"
#include "comm_common.cuh"

namespace lt {

constexpr int kMoeMaxRanks = 8;

struct RowGatherArgs {
  const __nv_bfloat16* src[kMoeMaxRanks];  // token buffers of every rank, [rows_r, cols] row-major
  const int2* slot_src;                    // [slots] {source rank, source row}; rank < 0: padding slot
  __nv_bfloat16* dst;                      // local slot buffer [slots, cols]
  uint32_t* flags;                         // one per 128-slot block
  uint32_t epoch;
  int slots, cols, n_blocks, n_comm;
  const __nv_bfloat16* zero_row;           // kGatherStageBytes of zeros: the source of padding slots
};

// Zeros that padding slots are "fetched" from, so that the rows of the slot buffer nobody owns are 0 and not stale
// shared memory (0 * NaN would poison the weight-gradient GEMMs that sum over whole 128-row blocks).
static __device__ __align__(128) uint8_t g_moe_zero_row[kGatherStageBytes];

// One thread per gather CTA: rows of a 128-slot block are fetched in batches that fill one 32 KB stage.
__device__ void gather_rows_cta(const RowGatherArgs& g, int* status) {
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
  const uint32_t row_bytes = uint32_t(g.cols) * 2u;
  int per_stage = int(kGatherStageBytes / row_bytes);
  if (per_stage < 1) return;  // rows wider than a stage are rejected by the host
  uint32_t use[kGatherStages];
  for (int s = 0; s < kGatherStages; ++s) use[s] = 0;

  for (int blk = blockIdx.x; blk < g.n_blocks; blk += g.n_comm) {
    const int r0 = blk * kBlockM;
    const int r1 = min(r0 + kBlockM, g.slots);
    int next_row = r0, issued = 0, stored = 0;
    int seg_row[kGatherStages], seg_rows[kGatherStages], seg_live[kGatherStages];
    bool ok = true;
    while (ok && (next_row < r1 || stored < issued)) {
      while (next_row < r1 && issued - stored < kGatherStages) {
        const int s = issued % kGatherStages;
        const int n = min(per_stage, r1 - next_row);
        tma_store_wait_read<0>();  // the stage's previous store has finished reading shared memory
        const uint32_t live = uint32_t(n);
        mbar_expect_tx(bb + 8u * s, live * row_bytes);
        for (int i = 0; i < n; ++i) {
          const int2 sr = g.slot_src[next_row + i];
          const __nv_bfloat16* from = sr.x >= 0 ? g.src[sr.x] + (long long)sr.y * g.cols : g.zero_row;
          bulk_g2s(sbase + s * kGatherStageBytes + i * row_bytes, from, row_bytes, bb + 8u * s);
        }
        seg_row[s] = next_row; seg_rows[s] = n; seg_live[s] = int(live);
        next_row += n;
        ++issued;
      }
      if (stored < issued) {
        const int s = stored % kGatherStages;
        if (seg_live[s]) {
          if (!mbar_wait(bb + 8u * s, use[s] & 1u, abort_flag, status, kStatusTimeoutFull)) { ok = false; break; }
          use[s]++;
          bulk_s2g(g.dst + (long long)seg_row[s] * g.cols, sbase + s * kGatherStageBytes, uint32_t(seg_rows[s]) * row_bytes);
          tma_store_commit();
        }
        ++stored;
      }
    }
    if (!ok) return;
    tma_store_wait<0>();
    asm volatile("fence.proxy.async.global;" ::: "memory");
    __threadfence();
    st_release_gpu(g.flags + blk, g.epoch);
  }
}

template <int BLOCK_N, int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_gather_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                       const RowGatherArgs g) {
  if (int(blockIdx.x) < g.n_comm) {
    gather_rows_cta(g, p.status);
    return;
  }
  FlagGate gate{g.flags, g.epoch, 2, -1};
  gemm_body<BLOCK_N, 0, B_MAJOR>(&tmA, &tmB, p, gate, NoDone(), g.n_comm);
}

template <int BLOCK_N, int B_MAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_gemm_scatter_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  gemm_body<BLOCK_N, 0, B_MAJOR>(&tmA, &tmB, p, NoGate(), NoDone());
}

template <class Kern>
static int set_smem(Kern kern, int bytes) {
  return cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace lt

extern "C" {

// C[slots, N] = rows gathered by slot table @ op(B[expert]).
//   src_ptrs[r]: rank r's token buffer [rows_r, K] bf16 (peer-mapped); slot_src: device int2 [slots] {rank, row};
//   group_of_mblk: device int [slots / 128] expert (local index) of every 128-slot block; slots is a multiple of 128;
//   B: [E, N, K] (b_major 0) or [E, K, N] (b_major 1) contiguous; slot_buf: local staging [slots, K]; flags: one uint32
//   per block, `epoch` grows with every call that reuses them; row_scale: optional fp32 [slots] applied in the epilogue.
int lt_moe_gather_gemm(const void* const* src_ptrs, int world, const void* slot_src, const int* group_of_mblk, int slots,
                       const void* B, int n_experts, int N, int K, int b_major, void* slot_buf, void* flags, unsigned epoch,
                       void* C, const float* row_scale, int n_comm, void* stream) {
  using namespace lt;
  if (slots == 0) return 0;
  if (slots % kBlockM != 0 || world < 1 || world > kMoeMaxRanks || K % 64 != 0 || N % 8 != 0 || K * 2 > kGatherStageBytes)
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  if (n_comm <= 0) n_comm = 8;
  int block_n = pick_block_n(slots, N, sms - n_comm);
  if (N % block_n != 0) block_n = (N % 128 == 0) ? 128 : 0;
  if (block_n == 0) return -int(kStatusBadArgument);
  GemmParams p{};
  p.M = slots; p.N = N; p.K = K;
  p.C = C; p.ldc = N; p.alpha = 1.f;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  p.raster = 2; p.rot = 0;
  p.group_of_mblk = group_of_mblk;
  p.b_group_rows = b_major == 0 ? N : K;
  p.row_scale = row_scale;
  RowGatherArgs g{};
  for (int r = 0; r < world; ++r) g.src[r] = static_cast<const __nv_bfloat16*>(src_ptrs[r]);
  g.slot_src = static_cast<const int2*>(slot_src);
  g.dst = static_cast<__nv_bfloat16*>(slot_buf);
  g.flags = static_cast<uint32_t*>(flags);
  g.epoch = epoch;
  g.slots = slots; g.cols = K; g.n_blocks = slots / kBlockM; g.n_comm = n_comm;
  {
    void* z = nullptr;
    LT_RETURN_IF_CUDA(cudaGetSymbolAddress(&z, g_moe_zero_row));
    g.zero_row = static_cast<const __nv_bfloat16*>(z);
  }
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, slot_buf, 2, (uint64_t)K, (uint64_t)slots, (uint64_t)K * 2, kBlockK, kBlockM, 1);
  if (r) return 1000 + r;
  if (b_major == 0) r = encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)n_experts * N, (uint64_t)K * 2, kBlockK, block_n, 1);
  else r = encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)n_experts * K, (uint64_t)N * 2, 64, kBlockK, 1);
  if (r) return 2000 + r;
  int grid = sms;
  if (grid - n_comm > p.num_tiles) grid = p.num_tiles + n_comm;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LT_MOE_GG(BN, BM)                                                                         \
  {                                                                                               \
    auto kern = moe_gather_gemm_kernel<BN, BM>;                                                   \
    int e = set_smem(kern, GemmCfg<BN>::kSmemBytes);                                              \
    if (e) return e;                                                                              \
    kern<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, st>>>(tmA, tmB, p, g);                    \
  }
  if (block_n == 256) { if (b_major) LT_MOE_GG(256, 1) else LT_MOE_GG(256, 0) }
  else { if (b_major) LT_MOE_GG(128, 1) else LT_MOE_GG(128, 0) }
#undef LT_MOE_GG
  LT_LAUNCH_CHECK();
  return 0;
}

// acc[dst_rank][dst_row, :] += row_weight[slot] * (A[slot, :] @ op(B[expert]))   for every slot with dst_rank >= 0.
//   A: local [slots, K] bf16; slot_dst: device int2 [slots] {rank, row}; acc_ptrs[r]: rank r's fp32 accumulator
//   [rows_r, N] (peer-mapped, zeroed by its owner before the ranks cross a barrier).
int lt_moe_gemm_scatter(const void* A, const int* group_of_mblk, int slots, const void* B, int n_experts, int N, int K,
                        int b_major, const void* slot_dst, const float* row_weight, const void* const* acc_ptrs, int world,
                        void* stream) {
  using namespace lt;
  if (slots == 0) return 0;
  if (slots % kBlockM != 0 || world < 1 || world > kMoeMaxRanks || K % 64 != 0 || N % 8 != 0) return -int(kStatusBadArgument);
  const int sms = sm_count();
  int block_n = pick_block_n(slots, N, sms);
  if (N % block_n != 0) block_n = (N % 128 == 0) ? 128 : 0;
  if (block_n == 0) return -int(kStatusBadArgument);
  GemmParams p{};
  p.M = slots; p.N = N; p.K = K;
  p.C = nullptr; p.ldc = N; p.alpha = 1.f; p.out_fp32 = 1;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  p.group_of_mblk = group_of_mblk;
  p.b_group_rows = b_major == 0 ? N : K;
  p.row_scale = row_weight;
  p.row_table = static_cast<const int2*>(slot_dst);
  for (int r = 0; r < world; ++r) p.acc_ptrs[r] = static_cast<float*>(const_cast<void*>(acc_ptrs[r]));
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, A, 2, (uint64_t)K, (uint64_t)slots, (uint64_t)K * 2, kBlockK, kBlockM, 1);
  if (r) return 1000 + r;
  if (b_major == 0) r = encode_tmap_2d(&tmB, B, 2, (uint64_t)K, (uint64_t)n_experts * N, (uint64_t)K * 2, kBlockK, block_n, 1);
  else r = encode_tmap_2d(&tmB, B, 2, (uint64_t)N, (uint64_t)n_experts * K, (uint64_t)N * 2, 64, kBlockK, 1);
  if (r) return 2000 + r;
  int grid = sms < p.num_tiles ? sms : p.num_tiles;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LT_MOE_GS(BN, BM)                                                                         \
  {                                                                                               \
    auto kern = moe_gemm_scatter_kernel<BN, BM>;                                                  \
    int e = set_smem(kern, GemmCfg<BN>::kSmemBytes);                                              \
    if (e) return e;                                                                              \
    kern<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, st>>>(tmA, tmB, p);                       \
  }
  if (block_n == 256) { if (b_major) LT_MOE_GS(256, 1) else LT_MOE_GS(256, 0) }
  else { if (b_major) LT_MOE_GS(128, 1) else LT_MOE_GS(128, 0) }
#undef LT_MOE_GS
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
