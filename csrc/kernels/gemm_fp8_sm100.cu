// Block-scaled fp8 (e4m3) GEMM for sm_100a:  C[M,N] = sum over 128-wide K blocks kb of
//     a_scale[kb][m] * b_scale[n / 128][kb] * (A8[m, kb] . B8[n, kb])
// A8 is [M, K] e4m3 with one fp32 scale per 1x128 block (activations), B8 is [N, K] e4m3 with one fp32 scale
// per 128x128 block (weights): the scaling layout of the fp8 training configuration.  The reference has no fp8
// GEMM (its cast kernels stop at fp16: src/backend/gpu_native/element/cast.cu); this is the B200 counterpart of
// the quantised Linear it sketches in python/litetorch/quantization.py.
//
// Two-level accumulation.  tcgen05.mma kind::f8f6f4 (128 x 128 x 32 per instruction, fp32 accumulate) computes
// the UNSCALED product of one K block into one of four 128-column TMEM buffers; the sixteen epilogue warps read
// that partial with tcgen05.ld and fold it into fp32 register accumulators with the block's scale, so that the
// scales are applied at full fp32 precision while the next K blocks are already running on the tensor core.
//   warp 0: TMA producer (128-byte-swizzled 128 x 128-byte tiles of A8 and B8, 6 stages)
//   warp 1: MMA issuer   (4 instructions per K block, commit -> stage free + partial ready)
//   warps 2-17: promotion + epilogue (4 warps per TMEM lane quarter, 32 columns each)
#include "lt_cuda.h"
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kF8BlockM = 128;
constexpr int kF8BlockN = 128;
constexpr int kF8BlockK = 128;   // elements == bytes
constexpr int kF8UmmaK = 32;
constexpr int kF8Stages = 6;
constexpr int kF8Bufs = 4;
constexpr int kF8EpiWarps = 16;           // four per TMEM lane quarter, 32 columns each
constexpr int kF8Threads = 64 + 32 * kF8EpiWarps;
constexpr int kF8TileBytes = kF8BlockM * kF8BlockK;
constexpr int kF8StageBytes = 2 * kF8TileBytes;
constexpr int kF8SmemBytes = kF8Stages * kF8StageBytes + 1024 + 512;

struct Fp8Params {
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  const float* a_scale;  // [K/128][M]
  const float* b_scale;  // [ceil(N/128)][K/128]
  const __nv_bfloat16* bias;
  int m_blocks, n_blocks, k_blocks, num_tiles;
  int* status;
};

__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Fp8Params p) {
  constexpr int S = kF8Stages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kF8StageBytes);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + kF8Bufs + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 2 * kF8Bufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  volatile int* issued_parity = reinterpret_cast<volatile int*>(tmem_holder + 2);  // [S]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      issued_parity[s] = -1;
    }
    for (int b = 0; b < kF8Bufs; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), kF8EpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kF8Bufs * kF8BlockN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        // M fastest: CTAs that run together share the B tile column and stream A once through L2
        const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, kF8StageBytes);
          issued_parity[stage] = int(phase);
          const uint32_t a_dst = smem_base + stage * kF8StageBytes;
          tma_load_2d(a_dst, &tmA, fb, kb * kF8BlockK, m_blk * kF8BlockM);
          tma_load_2d(a_dst + kF8TileBytes, &tmB, fb, kb * kF8BlockK, n_blk * kF8BlockN);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f8f6f4: a/b format 0 = e4m3, fp32 accumulate, both operands K-major
      constexpr uint32_t idesc = (1u << 4) | (uint32_t(kF8BlockN >> 3) << 17) | (uint32_t(kF8BlockM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t it = 0;  // running K-block count selects the TMEM buffer
      for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int buf = it % kF8Bufs;
          const uint32_t aphase = (it / kF8Bufs) & 1u;
          if (!mbar_wait(tempty_bar(buf), aphase ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * kF8StageBytes;
          const uint32_t b_addr = a_addr + kF8TileBytes;
          const uint32_t d_tmem = tmem_base + buf * kF8BlockN;
#pragma unroll
          for (int k = 0; k < kF8BlockK / kF8UmmaK; ++k) {
            const uint64_t adesc = make_smem_desc_sw128(a_addr + k * kF8UmmaK, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(b_addr + k * kF8UmmaK, 16, 1024);
            umma_f8_ss(d_tmem, adesc, bdesc, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          umma_commit(tfull_bar(buf));
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int part = (warp - 2) >> 2;      // which 32 columns of the tile
    uint32_t it = 0;
    bool alive = true;
    for (int tile = blockIdx.x; alive && tile < p.num_tiles; tile += gridDim.x) {
      const int m_blk = tile % p.m_blocks, n_blk = tile / p.m_blocks;
      const int row = m_blk * kF8BlockM + quarter * 32 + lane;
      const int srow = row < p.M ? row : p.M - 1;
      float acc[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = 0.f;
      float s_next = p.a_scale[srow] * p.b_scale[(long long)n_blk * p.k_blocks];
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        const float s = s_next;
        if (kb + 1 < p.k_blocks)
          s_next = p.a_scale[(long long)(kb + 1) * p.M + srow] * p.b_scale[(long long)n_blk * p.k_blocks + kb + 1];
        const int buf = it % kF8Bufs;
        const uint32_t aphase = (it / kF8Bufs) & 1u;
        const bool got = mbar_wait(tfull_bar(buf), aphase, abort_flag, p.status, kStatusTimeoutTmemFull);
        if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
        tc_fence_after();
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * kF8BlockN + part * 32, r);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(s, __uint_as_float(r[j]), acc[j]);
      }
      if (!alive || row >= p.M) continue;
      const int col0 = n_blk * kF8BlockN + part * 32;
      if (col0 >= p.N) continue;
      const bool vec = (col0 + 32 <= p.N) && (p.out_fp32 ? (p.ldc % 4 == 0) : (p.ldc % 8 == 0));
      if (p.bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) acc[j] += __bfloat162float(p.bias[col0 + j]);
      }
      if (p.out_fp32) {
        float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col0;
        if (vec) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            reinterpret_cast<float4*>(cp)[q] = make_float4(acc[q * 4], acc[q * 4 + 1], acc[q * 4 + 2], acc[q * 4 + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) cp[j] = acc[j];
        }
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
        if (vec) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16x2(acc[q * 8 + 0], acc[q * 8 + 1]);
            o.y = pack_bf16x2(acc[q * 8 + 2], acc[q * 8 + 3]);
            o.z = pack_bf16x2(acc[q * 8 + 4], acc[q * 8 + 5]);
            o.w = pack_bf16x2(acc[q * 8 + 6], acc[q * 8 + 7]);
            reinterpret_cast<uint4*>(cp)[q] = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) cp[j] = __float2bfloat16(acc[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      const int par = issued_parity[s];
      if (par < 0) continue;
      for (int spin = 0; spin < 20000; ++spin) {
        if (mbar_try_wait(full_bar(s), uint32_t(par))) break;
        __nanosleep(100);
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kF8Bufs * kF8BlockN);
  }
}

// Row-wise 1x128 quantisation of a bf16 matrix to e4m3 with the scales written K-block-major ([K/128][M]).
// One warp per (row, K block): amax by shuffle, scale = amax / 448, four values per lane.
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                   long long ldq, float* __restrict__ scale_t, int M, int K) {
  const int kblocks = K / 128;
  const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)M * kblocks) return;
  const int row = int(wid / kblocks), kb = int(wid % kblocks);
  const uint2 u = *reinterpret_cast<const uint2*>(x + (long long)row * ldx + kb * 128 + lane * 4);
  const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y);
  float amax = fmaxf(fmaxf(fabsf(f0.x), fabsf(f0.y)), fmaxf(fabsf(f1.x), fabsf(f1.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / scale;
  uint32_t packed;
  {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(f0.y * inv), "f"(f0.x * inv));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(f1.y * inv), "f"(f1.x * inv));
    packed = uint32_t(lo) | (uint32_t(hi) << 16);
  }
  *reinterpret_cast<uint32_t*>(q + (long long)row * ldq + kb * 128 + lane * 4) = packed;
  if (lane == 0) scale_t[(long long)kb * M + row] = scale;
}

}  // namespace lt

extern "C" {

// C[M,N] (bf16 or fp32) = block-scaled A8[M,K] * B8[N,K]^T (+ bias).  K must be a multiple of 128, lda/ldb (bytes ==
// elements) multiples of 16.  a_scale is [K/128][M] fp32, b_scale is [ceil(N/128)][K/128] fp32.
int lt_gemm_fp8_block(const void* A8, const void* B8, void* C, int M, int N, int K, long long lda, long long ldb,
                      long long ldc, const void* a_scale, const void* b_scale, int out_fp32, const void* bias,
                      int max_ctas, void* stream) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % kF8BlockK != 0 || lda % 16 != 0 || ldb % 16 != 0 || (reinterpret_cast<uintptr_t>(A8) & 15) ||
      (reinterpret_cast<uintptr_t>(B8) & 15))
    return -int(kStatusBadArgument);
  Fp8Params p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.a_scale = static_cast<const float*>(a_scale);
  p.b_scale = static_cast<const float*>(b_scale);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.m_blocks = (M + kF8BlockM - 1) / kF8BlockM;
  p.n_blocks = (N + kF8BlockN - 1) / kF8BlockN;
  p.k_blocks = K / kF8BlockK;
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.status = device_status_word();
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, A8, 1, (uint64_t)K, (uint64_t)M, (uint64_t)lda, kF8BlockK, kF8BlockM, 1);
  if (r) return 1000 + r;
  r = encode_tmap_2d(&tmB, B8, 1, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, kF8BlockK, kF8BlockN, 1);
  if (r) return 2000 + r;
  static bool configured = false;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8SmemBytes));
    configured = true;
  }
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > p.num_tiles) grid = p.num_tiles;
  gemm_fp8_kernel<<<grid, kF8Threads, kF8SmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, p);
  LT_LAUNCH_CHECK();
  return 0;
}

// q[M,K] e4m3 and scale_t[K/128][M] fp32 from x[M,K] bf16 (K a multiple of 128, ldx a multiple of 4).
int lt_quant_fp8_1x128(const void* x, long long ldx, void* q, long long ldq, void* scale_t, int M, int K, void* stream) {
  using namespace lt;
  if (M <= 0 || K <= 0) return 0;
  if (K % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return -int(kStatusBadArgument);
  const long long warps = (long long)M * (K / 128);
  const int wpb = 8;
  const long long blocks = (warps + wpb - 1) / wpb;
  quant_1x128_kernel<<<(unsigned)blocks, wpb * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(q), ldq, static_cast<float*>(scale_t), M, K);
  LT_LAUNCH_CHECK();
  return 0;
}

}  // extern "C"
