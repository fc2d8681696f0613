// Block-scaled fp8 (e4m3) GEMM on CTA pairs (tcgen05 cta_group::2, kind::f8f6f4): a cluster of two CTAs computes one
// 256 x 256 output tile.  Same arithmetic as gemm_fp8_sm100.cu (two-level accumulation: the tensor core produces the
// UNSCALED product of one 128-deep K block, the epilogue warps fold it into fp32 registers with
// a_scale[kb][m] * b_scale[n / 128][kb]); what changes is the operand traffic and the promotion bandwidth:
//   * each CTA stages its own 128 rows of A and HALF of the 256-column B tile (32 KB per K block instead of the
//     32 KB per 128 x 128 tile of the one-CTA kernel, i.e. half the bytes per MMA cycle);
//   * one K block is 512 tensor cycles per CTA (128 x 256 x 128), during which its 16 promotion warps read
//     128 x 256 fp32 from tensor memory: 64 columns per thread.
// Roles per CTA (576 threads): warp 0 TMA producer (both CTAs; bytes counted on the even CTA's barrier), warp 1 TMEM
// allocation in both CTAs and MMA issue in the even CTA, warps 2-17 promotion + epilogue of the CTA's own 128 rows.
// The reference has no fp8 GEMM that its ops use (cublasLtMatmul wrapper, src/backend/gpu_native/math/gemm.cu:122-155).
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kP8BlockM = 256, kP8BlockN = 256, kP8BlockK = 128, kP8UmmaK = 32;
constexpr int kP8Stages = 6;
constexpr int kP8Bufs = 2;
constexpr int kP8EpiWarps = 16;
constexpr int kP8Threads = 64 + 32 * kP8EpiWarps;
constexpr int kP8TileBytes = 128 * kP8BlockK;               // 128 rows x 128 bytes
constexpr int kP8StageBytes = 2 * kP8TileBytes;             // A rows + B half
constexpr int kP8SmemBytes = kP8Stages * kP8StageBytes + 1024 + 512;

struct Fp8PairParams {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  const float* a_scale;  // [K/128][M]
  const float* b_scale;  // [ceil(N/128)][K/128]
  const __nv_bfloat16* bias;
  int m_blocks, n_blocks, k_blocks, num_tiles;   // 256 x 256 tiles
  int* status;
};

__device__ __forceinline__ void umma_f8_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  const uint32_t z = 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}

// 18 warps: five on two of the four SM sub-partitions, whose 16 K registers each cap a thread at 96 registers.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kP8Threads, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8PairParams p) {
  constexpr int S = kP8Stages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kP8StageBytes);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                        // even CTA
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };                 // each CTA
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };             // each CTA
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + kP8Bufs + b); };  // even CTA: 32 warps arrive
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * kP8Bufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = (cta_rank == 0);
  const int pair_id = int(blockIdx.x) >> 1, pair_count = int(gridDim.x) >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < kP8Bufs; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 2 * kP8EpiWarps); }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < p.num_tiles; tile += pair_count) {
        const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
        const int m0 = m_blk * kP8BlockM + int(cta_rank) * 128;
        const int n0 = n_blk * kP8BlockN + int(cta_rank) * 128;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          const uint32_t fb = full_bar(stage);
          if (leader) mbar_expect_tx(fb, 2 * kP8StageBytes);
          const uint32_t a_dst = smem_base + stage * kP8StageBytes;
          tma_load_2d_pair(a_dst, &tmA, fb, kb * kP8BlockK, m0);
          tma_load_2d_pair(a_dst + kP8TileBytes, &tmB, fb, kb * kP8BlockK, n0);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // kind::f8f6f4: a/b format 0 = e4m3, fp32 accumulate, both operands K-major, M = 256 over the pair
      constexpr uint32_t idesc = (1u << 4) | (uint32_t(kP8BlockN >> 3) << 17) | (uint32_t(kP8BlockM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t it = 0;   // running K-block count selects the TMEM buffer
      for (int tile = pair_id; ok && tile < p.num_tiles; tile += pair_count) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int buf = it % kP8Bufs;
          const uint32_t aphase = (it / kP8Bufs) & 1u;
          if (!mbar_wait(tempty_bar(buf), aphase ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kP8StageBytes;
          const uint32_t b_addr = a_addr + kP8TileBytes;
          const uint32_t d_tmem = tmem_base + buf * kP8BlockN;
#pragma unroll
          for (int k = 0; k < kP8BlockK / kP8UmmaK; ++k)
            umma_f8_ss_pair(d_tmem, make_smem_desc_sw128(a_addr + k * kP8UmmaK, 16, 1024),
                            make_smem_desc_sw128(b_addr + k * kP8UmmaK, 16, 1024), idesc, k > 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(stage), 3);
          umma_commit_pair(tfull_bar(buf), 3);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;      // which 64 columns of the tile
    uint32_t it = 0;
    bool alive = true;
    for (int tile = pair_id; alive && tile < p.num_tiles; tile += pair_count) {
      const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
      const int row = m_blk * kP8BlockM + int(cta_rank) * 128 + quarter * 32 + lane;
      const int srow = row < p.M ? row : p.M - 1;
      const int n128 = min(n_blk * 2 + (part >> 1), (p.N + 127) / 128 - 1);   // b_scale row of these 64 columns
      float acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0.f;
      float s_next = p.a_scale[srow] * p.b_scale[(long long)n128 * p.k_blocks];
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        const float s = s_next;
        if (kb + 1 < p.k_blocks)
          s_next = p.a_scale[(long long)(kb + 1) * p.M + srow] * p.b_scale[(long long)n128 * p.k_blocks + kb + 1];
        const int buf = it % kP8Bufs;
        const uint32_t aphase = (it / kP8Bufs) & 1u;
        const bool got = mbar_wait(tfull_bar(buf), aphase, abort_flag, p.status, kStatusTimeoutTmemFull);
        if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kP8BlockN + part * 64;
        // 16 columns at a time: 64 accumulators + 16 loaded values stay inside the 96-register budget
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[16];
          tmem_ld_32x16(taddr + c * 16, r);
          tmem_ld_wait();
          if (c == 3) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_bar(buf), 0);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = fmaf(s, __uint_as_float(r[j]), acc[c * 16 + j]);
        }
      }
      if (!alive || row >= p.M) continue;
      const int col0 = n_blk * kP8BlockN + part * 64;
      if (col0 >= p.N) continue;
      const bool vec = (col0 + 64 <= p.N) && (p.out_fp32 ? (p.ldc % 4 == 0) : (p.ldc % 8 == 0));
      if (p.bias) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (col0 + j < p.N) acc[j] += __bfloat162float(p.bias[col0 + j]);
      }
      if (p.out_fp32) {
        float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
        if (vec) {
#pragma unroll
          for (int q = 0; q < 16; ++q)
            reinterpret_cast<float4*>(cp)[q] = make_float4(acc[q * 4], acc[q * 4 + 1], acc[q * 4 + 2], acc[q * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (col0 + j < p.N) cp[j] = acc[j];
        }
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
        if (vec) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 o;
            o.x = pack_bf16x2(acc[q * 8 + 0], acc[q * 8 + 1]);
            o.y = pack_bf16x2(acc[q * 8 + 2], acc[q * 8 + 3]);
            o.z = pack_bf16x2(acc[q * 8 + 4], acc[q * 8 + 5]);
            o.w = pack_bf16x2(acc[q * 8 + 6], acc[q * 8 + 7]);
            reinterpret_cast<uint4*>(cp)[q] = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j)
            if (col0 + j < p.N) cp[j] = __float2bfloat16(acc[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int spin = 0; spin < 20000; ++spin) __nanosleep(100);   // bounded grace period for copies in flight
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace lt

extern "C" {

// Same contract as lt_gemm_fp8_block; M > 128 and an even SM count are assumed by the caller's dispatch.
int lt_gemm_fp8_block_pair(const void* A8, const void* B8, void* C, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, const void* a_scale, const void* b_scale, int out_fp32, const void* bias,
                           void* stream) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % kP8BlockK != 0 || lda % 16 != 0 || ldb % 16 != 0 || (reinterpret_cast<uintptr_t>(A8) & 15) ||
      (reinterpret_cast<uintptr_t>(B8) & 15))
    return -int(kStatusBadArgument);
  Fp8PairParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.a_scale = static_cast<const float*>(a_scale);
  p.b_scale = static_cast<const float*>(b_scale);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.m_blocks = (M + kP8BlockM - 1) / kP8BlockM;
  p.n_blocks = (N + kP8BlockN - 1) / kP8BlockN;
  p.k_blocks = K / kP8BlockK;
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.status = device_status_word();
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, A8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kP8BlockK, 128, 1);
  if (r) return 1000 + r;
  r = encode_tmap_2d(&tmB, B8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, kP8BlockK, 128, 1);
  if (r) return 2000 + r;
  static bool configured = false;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(gemm_fp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kP8SmemBytes));
    configured = true;
  }
  int pairs = sm_count() / 2;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  gemm_fp8_pair_kernel<<<2 * pairs, kP8Threads, kP8SmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
