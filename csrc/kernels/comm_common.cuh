// Pieces shared by the fused compute + communication kernels: the flag gate that holds a GEMM tile back until the
// chunk it needs has landed, and the bulk asynchronous copies (never multicast) used by gather CTAs.
#pragma once
#include "gemm_sm100.cuh"

namespace lt {

struct FlagGate {
  const uint32_t* flags;
  uint32_t epoch;
  int gate_dim;
  int last;
  __device__ __forceinline__ bool operator()(int m_blk, int n_blk, int kb, int* status) {
    const int idx = gate_dim == 0 ? n_blk : (gate_dim == 1 ? kb : m_blk);
    if (idx == last) return true;
    if (!wait_flag_ge_gpu(flags + idx, epoch, status)) return false;
    asm volatile("fence.proxy.async.global;" ::: "memory");
    last = idx;
    return true;
  }
};

constexpr int kGatherStageBytes = 32768;
constexpr int kGatherStages = 5;

__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes) : "memory");
}

}  // namespace lt
