// Plain bf16 GEMM entry point on the tcgen05 / TMEM / TMA pipeline of gemm_sm100.cuh.
// Replaces the cuBLAS calls of the reference (src/backend/gpu_native/math/gemm.cu:3-189) and the
// backward GEMM pair of src/ops/linear.cpp:30-68, with bias / GELU / residual / accumulate epilogues.
#include "lt_cuda.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

namespace lt {

// MMA_KIND: 0 = bf16 / fp16 operands (kind::f16), 2 = fp32 operands as tf32, 3 = int8; one instruction kind per kernel.
template <int BLOCK_N, int A_MAJOR, int B_MAJOR, int MMA_KIND = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  gemm_body<BLOCK_N, A_MAJOR, B_MAJOR, MMA_KIND>(&tmA, &tmB, p, NoGate(), NoDone());
}

template <int BLOCK_N, int A_MAJOR, int B_MAJOR, int MMA_KIND = 0>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BLOCK_N>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BLOCK_N, A_MAJOR, B_MAJOR, MMA_KIND>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, st>>>(tmA, tmB, p);
  LT_LAUNCH_CHECK();
  return 0;
}

template <int A_MAJOR, int B_MAJOR, int MMA_KIND = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  gemm_body_pair<A_MAJOR, B_MAJOR, MMA_KIND>(&tmA, &tmB, p, NoGate(), NoDone());
}

template <int A_MAJOR, int B_MAJOR, int MMA_KIND = 0>
static int launch_gemm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t st) {
  static bool configured = false;
  auto kern = gemm_bf16_pair_kernel<A_MAJOR, B_MAJOR, MMA_KIND>;
  if (!configured) {
    LT_RETURN_IF_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes));
    configured = true;
  }
  kern<<<grid, kGemmThreads, kPairSmemBytes, st>>>(tmA, tmB, p);
  LT_LAUNCH_CHECK();
  return 0;
}

// 0: never use CTA pairs; 1: where the cost model prefers them; 2: wherever the shape allows.
static std::atomic<int> g_pair_mode{1};
int gemm_pair_mode() { return g_pair_mode.load(); }

// Workspace of the split tail, one per (device, stream): launches on one stream are serialised, so the partial
// tiles and the flags of one launch are consumed before the next launch writes them.
struct SplitWs {
  float* ws = nullptr;
  unsigned* flags = nullptr;
};
constexpr int kSplitSlots = 160;                                   // >= SM count: at most one partial per CTA
constexpr size_t kSplitSlotBytes = size_t(kBlockM) * 256 * 4;      // one 128 x 256 fp32 partial
static std::mutex g_split_mu;
static std::map<std::pair<int, cudaStream_t>, SplitWs> g_split_ws;
static std::atomic<int> g_split_enabled{1};

static bool get_split_ws(cudaStream_t st, SplitWs* out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(g_split_mu);
  auto key = std::make_pair(dev, st);
  auto it = g_split_ws.find(key);
  if (it != g_split_ws.end()) { *out = it->second; return out->ws != nullptr; }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return false;   // no allocation while a graph is being captured: this launch runs without the split
  }
  SplitWs w;
  void* base = nullptr;
  if (cudaMalloc(&base, kSplitSlots * kSplitSlotBytes + kSplitSlots * 4 * sizeof(unsigned)) != cudaSuccess) {
    cudaGetLastError();
    g_split_ws[key] = SplitWs{};
    return false;
  }
  w.ws = static_cast<float*>(base);
  w.flags = reinterpret_cast<unsigned*>(static_cast<char*>(base) + kSplitSlots * kSplitSlotBytes);
  if (cudaMemsetAsync(w.flags, 0, kSplitSlots * 4 * sizeof(unsigned), st) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(base);
    g_split_ws[key] = SplitWs{};
    return false;
  }
  g_split_ws[key] = w;
  *out = w;
  return true;
}

}  // namespace lt

extern "C" {

// 0: one CTA per tile only; 1 (default): CTA pairs (256 x 256 tiles on cta_group::2) where the cost model prefers
// them; 2: CTA pairs for every shape.
void lt_gemm_set_pair_mode(int mode) { lt::g_pair_mode.store(mode < 0 ? 0 : (mode > 2 ? 2 : mode)); }

// 1 (default): GEMMs whose last wave fills only part of the GPU cut the tiles of that wave along K.  0: off.
void lt_gemm_set_tail_split(int enable) { lt::g_split_enabled.store(enable ? 1 : 0); }

// C[M,N] = epilogue(alpha * op(A) * op(B)).  See gemm_sm100.cuh for the operand layouts.
// lda/ldb/ldc/ldr are pitches in elements. block_n: 0 = choose, else 128 or 256. max_ctas: 0 = one per SM.
// Returns 0, a cudaError_t, or 1000+/2000+ CUresult when a tensor map could not be encoded.
static int gemm_launch(int kind, const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                       long long ldr, int act, int accumulate, float alpha, int block_n, int max_ctas, void* stream,
                       const float* a_scale = nullptr, const float* b_scale = nullptr);

int lt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                 long long ldr, int act, int accumulate, float alpha, int block_n, int max_ctas, void* stream) {
  return gemm_launch(0, A, B, C, M, N, K, lda, ldb, ldc, a_major, b_major, out_fp32, bias, residual, ldr, act, accumulate, alpha,
                     block_n, max_ctas, stream);
}

// The same GEMM for fp16 operands (kind 1: any operand layout, C bf16 or fp32), for fp32 operands on the tensor cores
// as tf32 (kind 2: both operands K-major, i.e. a_major = b_major = 0, K a multiple of 4, C fp32) and for signed int8
// operands (kind 3: both K-major, K a multiple of 16, C = alpha * integer sums as fp32; the reference's
// w8a8_matmul_kernel, src/backend/gpu_native/nn/nn_kernels.cu:1314-1337).  bias / residual
// stay bf16.  Takes the place of the reference's cublasHgemm / cublasSgemm-with-TF32 paths
// (src/backend/gpu_native/math/gemm.cu:3-47, 75-120).
int lt_gemm_typed(int kind, const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                  long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                  long long ldr, int act, int accumulate, float alpha, void* stream) {
  using namespace lt;
  if (kind < 0 || kind > 3) return -int(kStatusBadArgument);
  if (kind == 3) {
    // signed int8 operands, both K-major, C = alpha * (int32 sums) as fp32; rows seen as 2-byte units of half the extent
    if (a_major != 0 || b_major != 0 || !out_fp32 || (K & 15) || (lda & 15) || (ldb & 15) || bias || residual) return -int(kStatusBadArgument);
    return gemm_launch(3, A, B, C, M, N, K / 2, lda / 2, ldb / 2, ldc, 0, 0, 1, nullptr, nullptr, 0, 0, accumulate, alpha, 0, 0, stream);
  }
  if (kind == 2) {
    if (a_major != 0 || b_major != 0 || !out_fp32 || (K & 3) || (lda & 3) || (ldb & 3)) return -int(kStatusBadArgument);
    // fp32 rows seen as rows of 2-byte units: twice the K extent and twice the pitches
    return gemm_launch(2, A, B, C, M, N, 2 * K, 2 * lda, 2 * ldb, ldc, 0, 0, 1, bias, residual, ldr, act, accumulate, alpha, 0, 0, stream);
  }
  return gemm_launch(kind, A, B, C, M, N, K, lda, ldb, ldc, a_major, b_major, out_fp32, bias, residual, ldr, act, accumulate,
                     alpha, 0, 0, stream);
}

// C = epilogue((A[M, K] @ B[N, K]^T) * a_scale[row] * b_scale[column]) for e4m3 operands, both K-major, on tcgen05
// kind::f8f6f4 (twice the bf16 MMA rate): the whole K extent accumulates in tensor memory and the scales are applied
// once in the epilogue, so the kernel is the bf16 CTA-pair kernel with another instruction.  Scales per row of the
// activations and per row of the weight (its output channel) are what per-token / per-channel fp8 training recipes use;
// the 1x128 / 128x128 block-scaled variant (gemm_fp8_sm100.cu) pays a tensor-memory round trip per 128-deep K block
// instead.  K a multiple of 16, pitches in elements (bytes).  C bf16 or fp32; bias / residual bf16.
int lt_gemm_e4m3(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, long long ldc,
                 int out_fp32, const float* a_scale, const float* b_scale, const void* bias, const void* residual,
                 long long ldr, int act, float alpha, void* stream) {
  if ((K & 15) || (lda & 15) || (ldb & 15)) return -int(lt::kStatusBadArgument);
  // e4m3 rows seen as rows of 2-byte units of half the extent (the copy is byte-identical)
  return gemm_launch(4, A, B, C, M, N, K / 2, lda / 2, ldb / 2, ldc, 0, 0, out_fp32, bias, residual, ldr, act, 0, alpha, 0, 0, stream,
                     a_scale, b_scale);
}

static int gemm_launch(int kind, const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                       long long ldr, int act, int accumulate, float alpha, int block_n, int max_ctas, void* stream,
                       const float* a_scale, const float* b_scale) {
  using namespace lt;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda * 2) % 16 != 0 || (ldb * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -int(kStatusBadArgument);
  const int sms = sm_count();
  // int8: integer accumulators are converted in the one-CTA kernel's epilogue; no K split (its workspace holds floats)
  const bool split_on = kind != 3 && g_split_enabled.load() != 0;
  const int pair_mode = kind == 3 ? 0 : g_pair_mode.load();
  if (pair_mode > 0 && block_n != 128 && (max_ctas <= 0 || max_ctas >= sms)) {
    const double c256 = wave_cost(M, N, K, sms, 256), c128 = wave_cost(M, N, K, sms, 128);
    const double single = c256 < c128 ? c256 : c128;
    if (pair_mode == 2 || pair_cost(M, N, K, sms, split_on) < single) {
      GemmParams q{};
      q.kind = kind;
      q.M = M; q.N = N; q.K = K;
      q.C = C; q.ldc = ldc; q.out_fp32 = out_fp32;
      q.bias = static_cast<const __nv_bfloat16*>(bias);
      q.residual = static_cast<const __nv_bfloat16*>(residual);
      q.ldr = ldr; q.act = act; q.accumulate = accumulate; q.alpha = alpha;
      q.a_scale = a_scale; q.b_scale = b_scale;
      q.status = device_status_word();
      fill_tiles(q, kPairBlockN);
      fill_pair_tiles(q);
      CUtensorMap tmA, tmB;
      int r = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_major, b_major, kPairBlockN / 2);
      if (r) return r;
      int pairs = sms / 2;
      if (pairs > q.num_tiles) pairs = q.num_tiles;
      cudaStream_t st = static_cast<cudaStream_t>(stream);
      if (split_on) {
        const int split = pair_tail_split(q.num_tiles, q.k_blocks, pairs);
        SplitWs w;
        if (split > 1 && get_split_ws(st, &w)) {
          q.dp_tiles = (q.num_tiles / pairs) * pairs;
          q.sk_tiles = q.num_tiles - q.dp_tiles;
          q.sk_split = split;
          q.sk_ws = w.ws;
          q.sk_flags = w.flags;
        }
      }
      if (kind == 2) return launch_gemm_pair<0, 0, 2>(tmA, tmB, q, 2 * pairs, st);   // tf32: both operands K-major
      if (kind == 4) return launch_gemm_pair<0, 0, 4>(tmA, tmB, q, 2 * pairs, st);   // e4m3: both operands K-major
      const int key2 = (a_major ? 2 : 0) | (b_major ? 1 : 0);
      switch (key2) {
        case 0: return launch_gemm_pair<0, 0>(tmA, tmB, q, 2 * pairs, st);
        case 1: return launch_gemm_pair<0, 1>(tmA, tmB, q, 2 * pairs, st);
        case 2: return launch_gemm_pair<1, 0>(tmA, tmB, q, 2 * pairs, st);
        default: return launch_gemm_pair<1, 1>(tmA, tmB, q, 2 * pairs, st);
      }
    }
  }
  if (block_n != 128 && block_n != 256) block_n = split_on ? pick_block_n_split(M, N, K, sms) : pick_block_n(M, N, sms);
  GemmParams p{};
  p.kind = kind;
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr; p.act = act; p.accumulate = accumulate; p.alpha = alpha;
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.status = device_status_word();
  fill_tiles(p, block_n);
  CUtensorMap tmA, tmB;
  int r = make_operand_maps(&tmA, &tmB, A, B, M, N, K, lda, ldb, a_major, b_major, block_n);
  if (r) return r;
  int grid = sms;
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (grid > p.num_tiles) grid = p.num_tiles;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (split_on) {
    const int split = tail_split(p.num_tiles, p.k_blocks, grid);
    SplitWs w;
    if (split > 1 && get_split_ws(st, &w)) {
      p.dp_tiles = (p.num_tiles / grid) * grid;
      p.sk_tiles = p.num_tiles - p.dp_tiles;
      p.sk_split = split;
      p.sk_ws = w.ws;
      p.sk_flags = w.flags;
    }
  }
  if (kind == 2) return block_n == 256 ? launch_gemm<256, 0, 0, 2>(tmA, tmB, p, grid, st) : launch_gemm<128, 0, 0, 2>(tmA, tmB, p, grid, st);
  if (kind == 3) return block_n == 256 ? launch_gemm<256, 0, 0, 3>(tmA, tmB, p, grid, st) : launch_gemm<128, 0, 0, 3>(tmA, tmB, p, grid, st);
  if (kind == 4) return block_n == 256 ? launch_gemm<256, 0, 0, 4>(tmA, tmB, p, grid, st) : launch_gemm<128, 0, 0, 4>(tmA, tmB, p, grid, st);
  const int key = (block_n == 256 ? 4 : 0) | (a_major ? 2 : 0) | (b_major ? 1 : 0);
  switch (key) {
    case 0: return launch_gemm<128, 0, 0>(tmA, tmB, p, grid, st);
    case 1: return launch_gemm<128, 0, 1>(tmA, tmB, p, grid, st);
    case 2: return launch_gemm<128, 1, 0>(tmA, tmB, p, grid, st);
    case 3: return launch_gemm<128, 1, 1>(tmA, tmB, p, grid, st);
    case 4: return launch_gemm<256, 0, 0>(tmA, tmB, p, grid, st);
    case 5: return launch_gemm<256, 0, 1>(tmA, tmB, p, grid, st);
    case 6: return launch_gemm<256, 1, 0>(tmA, tmB, p, grid, st);
    default: return launch_gemm<256, 1, 1>(tmA, tmB, p, grid, st);
  }
}

}  // extern "C"
