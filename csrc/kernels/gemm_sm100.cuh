// Persistent, warp-specialised bf16 GEMM for sm_100a, shared by the plain GEMM entry point and the
// fused communication variants (all-gather -> GEMM, GEMM -> reduce-scatter).
//
//   C[M,N] = epilogue(alpha * A * B)   with fp32 accumulation in tensor memory
//
// Operand layouts (element type bf16):
//   A_MAJOR = 0: A is stored [M, K] row-major (K contiguous);   A_MAJOR = 1: A is stored [K, M] row-major.
//   B_MAJOR = 0: B is stored [N, K] row-major (K contiguous);   B_MAJOR = 1: B is stored [K, N] row-major.
// so (0,0) is x @ W^T of a Linear layer, (0,1) is dY @ W, (1,1) is dY^T @ X.
//
// Pipeline per CTA (192 threads, one CTA per SM, grid-stride over output tiles):
//   warp 0   : TMA producer   (cp.async.bulk.tensor, 128-byte swizzle, mbarrier complete_tx)
//   warp 1   : MMA issuer     (tcgen05.mma 128 x BLOCK_N x 16, accumulators double-buffered in TMEM)
//   warps 2-5: epilogue       (tcgen05.ld -> registers -> bias / GELU / residual / accumulate -> global)
// The epilogue of tile i overlaps the main loop of tile i+1 through the two TMEM accumulator buffers.
//
// Hooks: a `TileGate` functor lets a fused variant delay a tile until the data it needs has arrived
// (all-gather -> GEMM) and a `TileDone` functor lets it publish a finished tile (GEMM -> reduce-scatter).
#pragma once
#include "common/host.h"
#include "common/ptx.cuh"

namespace lt {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;

struct GemmParams {
  // Operand element kind: 0 = bf16, 1 = fp16 (both kind::f16), 2 = fp32 used as tf32 (kind::tf32), 3 = signed int8
  // (kind::i8, 32-bit integer accumulators that the epilogue converts to float; one-CTA kernel only), 4 = e4m3 (kind::f8f6f4,
  // scaled per row of A and per row of B through a_scale / b_scale).  For tf32 / int8 / e4m3 the
  // host describes the operands to TMA as 2-byte elements of twice the K extent (the copy is byte-identical) and
  // K below counts those 2-byte units, so the tiling, the 128-byte swizzled stage rows and the 32-byte descriptor
  // step per MMA are the same for every kind; only the instruction and the format bits of its descriptor differ.
  int kind;
  int M, N, K;
  void* C;
  long long ldc;
  int out_fp32;
  const __nv_bfloat16* bias;      // [N] or nullptr
  const __nv_bfloat16* residual;  // [M, N] (pitch ldr) or nullptr
  long long ldr;
  int act;         // 0 none, 1 GELU(tanh)
  int accumulate;  // C += result
  float alpha;
  int m_blocks, n_blocks, k_blocks, num_tiles;
  int group_m;  // raster group height (tiles)
  // Tile order: 0 = grouped raster (L2 friendly; groups of group_m M blocks, starting at group `rot`); 1 = all M blocks of one N block before the next N block,
  // starting at N block `rot`; 2 = all N blocks of one M block before the next, starting at M block `rot`.
  // Modes 1 and 2 let a fused all-gather deliver the gathered operand in the order the tiles consume it.
  int raster, rot;
  int k_rot;  // the K loop starts at k-block k_rot and wraps around
  int* status;
  // Scatter mode (GEMM -> reduce-scatter): when rows_per_rank > 0 the tile rows are not written to C but to the
  // staging buffer of the rank that owns them, peer_C[owner] + (src_rank * rows_per_rank + local_row) * ldc.
  void* peer_C[8];
  int rows_per_rank, src_rank;
  // Grouped GEMM (mixture of experts): rows are grouped by expert in blocks of 128; m block i uses the B operand of
  // expert group_of_mblk[i], i.e. B rows are offset by group * b_group_rows (nullptr: plain GEMM).
  const int* group_of_mblk;
  int b_group_rows;
  // Per-row epilogue extras: multiply row r by row_scale[r]; combine mode: instead of storing, add the row (times
  // row_scale) into the fp32 accumulator of the rank that owns the token, acc_ptrs[dst_rank] + dst_row * ldc, with
  // red.add (peer memory over NVLink); row_table[r] = {dst_rank, dst_row}, dst_rank < 0 marks a padding row.
  const float* row_scale;
  const int2* row_table;
  float* acc_ptrs[8];
  // Split tail: tiles [0, dp_tiles) are computed whole, one per CTA per wave; when the last wave would leave most SMs
  // idle, each of the remaining sk_tiles tiles is cut along K into sk_split parts that run on different CTAs.  Parts
  // 1..sk_split-1 dump their fp32 accumulators into sk_ws and bump sk_flags[tile * 4 + lane quarter]; part 0 waits for
  // them (bounded), adds them to its own accumulator and runs the normal epilogue.  sk_split <= 1: no split.
  int dp_tiles, sk_tiles, sk_split;
  float* sk_ws;          // [sk_tiles][sk_split - 1][BLOCK_N / 32][8][128 rows][4]
  unsigned* sk_flags;    // [sk_tiles][4], zero between launches
  // Dequantisation of 8-bit operands, applied to the accumulator before bias / residual: row r times a_scale[r], column c
  // times b_scale[c] (fp32, nullptr: 1).
  const float* a_scale;
  const float* b_scale;
};

struct WorkItem {
  int tile, kb0, kb1;
  int split;   // -1: whole tile; 0: owner of a split tile; > 0: contributor
  int slot;    // index of the split tile (0 .. sk_tiles-1)
};

// The i-th piece of work of CTA cta_id out of cta_count.
__device__ __forceinline__ bool get_item(const GemmParams& p, int cta_id, int cta_count, int i, WorkItem& w) {
  const int tile = cta_id + i * cta_count;
  if (tile < p.dp_tiles) {
    w.tile = tile; w.kb0 = 0; w.kb1 = p.k_blocks; w.split = -1; w.slot = 0;
    return true;
  }
  if (p.sk_split > 1 && i == p.dp_tiles / cta_count && cta_id < p.sk_tiles * p.sk_split) {
    const int t = cta_id % p.sk_tiles, part = cta_id / p.sk_tiles;
    w.tile = p.dp_tiles + t;
    w.kb0 = int((long long)part * p.k_blocks / p.sk_split);
    w.kb1 = int((long long)(part + 1) * p.k_blocks / p.sk_split);
    w.split = part; w.slot = t;
    return true;
  }
  return false;
}

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int kTmemCols = 2 * BLOCK_N;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kBarrierBytes;
};

struct NoGate {
  __device__ __forceinline__ bool operator()(int, int, int, int*) const { return true; }
};
struct NoDone {
  __device__ __forceinline__ void fence() const {}                 // every epilogue lane, after its stores
  __device__ __forceinline__ void operator()(int, int) const {}    // one lane per epilogue warp, after the fence
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_blk, int& n_blk) {
  if (p.raster == 1) {
    m_blk = tile % p.m_blocks;
    n_blk = (tile / p.m_blocks + p.rot) % p.n_blocks;
    return;
  }
  if (p.raster == 2) {
    n_blk = tile % p.n_blocks;
    m_blk = (tile / p.n_blocks + p.rot) % p.m_blocks;
    return;
  }
  const int per_group = p.group_m * p.n_blocks;
  int group = tile / per_group;
  const int in_group = tile - group * per_group;   // position inside the group, taken before the group is rotated
  if (p.rot > 0) {   // groups start at group `rot` and wrap (only set when every group is full)
    const int n_groups = p.m_blocks / p.group_m;
    group += p.rot;
    if (group >= n_groups) group -= n_groups;
  }
  const int first_m = group * p.group_m;
  const int rows = min(p.m_blocks - first_m, p.group_m);
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

// One 32-column slice of one output row.
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, int row, int col0, const uint32_t (&r)[32]) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = (p.kind == 3 ? float(int(r[j])) : __uint_as_float(r[j])) * p.alpha;
  const bool full = (col0 + 32 <= p.N);
  const int ncols = full ? 32 : (p.N - col0);
  if (p.a_scale) {
    const float as = __ldg(p.a_scale + row);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= as;
  }
  if (p.b_scale) {
    if (full && (reinterpret_cast<uintptr_t>(p.b_scale) & 15) == 0) {
      const float4* b4 = reinterpret_cast<const float4*>(p.b_scale + col0);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 f = __ldg(b4 + q);
        v[q * 4 + 0] *= f.x; v[q * 4 + 1] *= f.y; v[q * 4 + 2] *= f.z; v[q * 4 + 3] *= f.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (j < ncols) v[j] *= __ldg(p.b_scale + col0 + j);
    }
  }
  if (p.bias) {
    if (full) {
      const uint4* b4 = reinterpret_cast<const uint4*>(p.bias + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 u = __ldg(b4 + q);
        float2 f;
        f = unpack_bf16x2(u.x); v[q * 8 + 0] += f.x; v[q * 8 + 1] += f.y;
        f = unpack_bf16x2(u.y); v[q * 8 + 2] += f.x; v[q * 8 + 3] += f.y;
        f = unpack_bf16x2(u.z); v[q * 8 + 4] += f.x; v[q * 8 + 5] += f.y;
        f = unpack_bf16x2(u.w); v[q * 8 + 6] += f.x; v[q * 8 + 7] += f.y;
      }
    } else {
      _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __bfloat162float(p.bias[col0 + j]);
    }
  }
  if (p.act == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
  }
  if (p.residual) {
    const __nv_bfloat16* rp = p.residual + (long long)row * p.ldr + col0;
    if (full && (p.ldr % 8 == 0)) {
      const uint4* r4 = reinterpret_cast<const uint4*>(rp);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 u = r4[q];
        float2 f;
        f = unpack_bf16x2(u.x); v[q * 8 + 0] += f.x; v[q * 8 + 1] += f.y;
        f = unpack_bf16x2(u.y); v[q * 8 + 2] += f.x; v[q * 8 + 3] += f.y;
        f = unpack_bf16x2(u.z); v[q * 8 + 4] += f.x; v[q * 8 + 5] += f.y;
        f = unpack_bf16x2(u.w); v[q * 8 + 6] += f.x; v[q * 8 + 7] += f.y;
      }
    } else {
      _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) v[j] += __bfloat162float(rp[j]);
    }
  }
  if (p.row_scale) {
    const float rs = p.row_scale[row];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= rs;
  }
  if (p.row_table) {
    const int2 dst = p.row_table[row];
    if (dst.x < 0) return;
    float* ap = p.acc_ptrs[dst.x] + (long long)dst.y * p.ldc + col0;
    if (full) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(ap + q * 4), "f"(v[q * 4]), "f"(v[q * 4 + 1]),
                     "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3]) : "memory");
    } else {
      _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) atomicAdd(ap + j, v[j]);
    }
    return;
  }
  void* c_base = p.C;
  if (p.rows_per_rank > 0) {
    const int owner = row / p.rows_per_rank;
    c_base = p.peer_C[owner];
    row = p.src_rank * p.rows_per_rank + (row - owner * p.rows_per_rank);
  }
  if (p.out_fp32) {
    float* cp = reinterpret_cast<float*>(c_base) + (long long)row * p.ldc + col0;
    if (full && (p.ldc % 4 == 0)) {
      float4* c4 = reinterpret_cast<float4*>(cp);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float4 o = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        if (p.accumulate) {
          float4 old = c4[q];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        c4[q] = o;
      }
    } else {
      _Pragma("unroll") for (int j = 0; j < 32; ++j) if (j < ncols) cp[j] = p.accumulate ? cp[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(c_base) + (long long)row * p.ldc + col0;
    if (full && (p.ldc % 8 == 0)) {
      uint4* c4 = reinterpret_cast<uint4*>(cp);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (p.accumulate) {
          uint4 old = c4[q];
          float2 f;
          f = unpack_bf16x2(old.x); v[q * 8 + 0] += f.x; v[q * 8 + 1] += f.y;
          f = unpack_bf16x2(old.y); v[q * 8 + 2] += f.x; v[q * 8 + 3] += f.y;
          f = unpack_bf16x2(old.z); v[q * 8 + 4] += f.x; v[q * 8 + 5] += f.y;
          f = unpack_bf16x2(old.w); v[q * 8 + 6] += f.x; v[q * 8 + 7] += f.y;
        }
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        c4[q] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j >= ncols) break;
        float o = v[j];
        if (p.accumulate) o += __bfloat162float(cp[j]);
        cp[j] = __float2bfloat16(o);
      }
    }
  }
}

// The body shared by all GEMM kernels. `gate(m_blk, n_blk, kb, status)` is called by the producer
// before it loads k-block kb of a tile and returns false if a bounded wait ran out; `done(m_blk, n_blk)`
// is called by one thread of each epilogue warp after the warp's rows of a tile are in global memory.
// MMA_KIND selects the instruction a kernel is built around: 0 = kind::f16 (bf16 and fp16 operands, told apart by the
// format bits of the run-time instruction descriptor), 2 = kind::tf32, 3 = kind::i8, 4 = kind::f8f6f4 with e4m3 operands.  It is a template parameter and
// not a run-time branch on purpose: a kernel that contains tcgen05.mma instructions of more than one kind ran its
// bf16 MMAs at half rate (measured: 1000 instead of 512 cycles per 256 x 256 x 64 block with no loads in flight).
template <int BLOCK_N, int A_MAJOR, int B_MAJOR, int MMA_KIND = 0, class TileGate, class TileDone>
__device__ __forceinline__ void gemm_body(const CUtensorMap* tmA, const CUtensorMap* tmB, const GemmParams& p,
                                          TileGate gate, TileDone done, int cta_first = 0) {
  // CTAs [0, cta_first) of the grid belong to another role of a fused kernel; the GEMM uses the rest.
  const int cta_id = int(blockIdx.x) - cta_first;
  const int cta_count = int(gridDim.x) - cta_first;
  using Cfg = GemmCfg<BLOCK_N>;
  constexpr int S = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::kStageBytes);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * S + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * S + 2 + b); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
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
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      for (int i = 0; ok && get_item(p, cta_id, cta_count, i, w); ++i) {
        int m_blk, n_blk;
        tile_coords(p, w.tile, m_blk, n_blk);
        for (int kl = w.kb0; kl < w.kb1; ++kl) {
          int kb = kl + p.k_rot;   // k_rot is only used with whole tiles
          if (kb >= p.k_blocks) kb -= p.k_blocks;
          if (!gate(m_blk, n_blk, kb, p.status)) { *abort_flag = 1; ok = false; break; }
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kStatusTimeoutEmpty)) { ok = false; break; }
          const uint32_t fb = full_bar(stage);
          mbar_expect_tx(fb, Cfg::kStageBytes);
          issued_parity[stage] = int(phase);
          const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
          const uint32_t b_dst = a_dst + Cfg::kABytes;
          if (A_MAJOR == 0) {
            tma_load_2d(a_dst, tmA, fb, kb * kBlockK, m_blk * kBlockM);
          } else {
#pragma unroll
            for (int i = 0; i < kBlockM / 64; ++i)
              tma_load_2d(a_dst + i * (64 * kBlockK * 2), tmA, fb, m_blk * kBlockM + i * 64, kb * kBlockK);
          }
          const int b_off = p.group_of_mblk ? p.group_of_mblk[m_blk] * p.b_group_rows : 0;
          if (B_MAJOR == 0) {
            tma_load_2d(b_dst, tmB, fb, kb * kBlockK, b_off + n_blk * BLOCK_N);
          } else {
#pragma unroll
            for (int i = 0; i < BLOCK_N / 64; ++i)
              tma_load_2d(b_dst + i * (64 * kBlockK * 2), tmB, fb, n_blk * BLOCK_N + i * 64, b_off + kb * kBlockK);
          }
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = MMA_KIND == 3 ? make_idesc_i8(kBlockM, BLOCK_N)
                             : MMA_KIND == 4 ? make_idesc_e4m3(kBlockM, BLOCK_N)
                                             : make_idesc_f16(kBlockM, BLOCK_N, MMA_KIND == 2 ? 2 : (p.kind == 1 ? 0 : 1), A_MAJOR, B_MAJOR);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkItem w;
      for (int it = 0; ok && get_item(p, cta_id, cta_count, it, w); ++it) {
        const int buf = it & 1;
        const uint32_t aphase = (it >> 1) & 1;
        if (!mbar_wait(tempty_bar(buf), aphase ^ 1u, abort_flag, p.status, kStatusTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BLOCK_N;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kStatusTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + Cfg::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t adesc = (A_MAJOR == 0) ? make_smem_desc_sw128(a_addr + k * (kUmmaK * 2), 16, 1024)
                                                  : make_smem_desc_sw128(a_addr + k * (kUmmaK * 128), 64 * kBlockK * 2, 1024);
            const uint64_t bdesc = (B_MAJOR == 0) ? make_smem_desc_sw128(b_addr + k * (kUmmaK * 2), 16, 1024)
                                                  : make_smem_desc_sw128(b_addr + k * (kUmmaK * 128), 64 * kBlockK * 2, 1024);
            if constexpr (MMA_KIND == 2) umma_tf32_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
            else if constexpr (MMA_KIND == 3) umma_i8_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
            else if constexpr (MMA_KIND == 4) umma_e4m3_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
            else umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    WorkItem w;
    for (int it = 0; get_item(p, cta_id, cta_count, it, w); ++it) {
      int m_blk, n_blk;
      tile_coords(p, w.tile, m_blk, n_blk);
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1;
      const bool got = mbar_wait(tfull_bar(buf), aphase, abort_flag, p.status, kStatusTimeoutTmemFull);
      if (!__all_sync(0xffffffffu, got)) break;
      tc_fence_after();
      const int row = m_blk * kBlockM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * BLOCK_N;
      if (w.split > 0) {
        // contributor of a split tile: raw accumulators to the workspace, then one arrival per warp
        float* ws = p.sk_ws + ((long long)(w.slot * (p.sk_split - 1) + (w.split - 1)) * (BLOCK_N / 32)) * (kBlockM * 32) +
                    (quarter * 32 + lane) * 4;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {
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
          mbar_arrive(tempty_bar(buf));
          red_add_release_gpu(p.sk_flags + w.slot * 4 + quarter, 1u);
        }
        continue;
      }
      bool parts_ok = true;
      if (w.split == 0) {
        // owner of a split tile: the other parts of this lane quarter must have landed
        int okf = 1;
        if (lane == 0) {
          okf = wait_flag_ge_gpu(p.sk_flags + w.slot * 4 + quarter, uint32_t(p.sk_split - 1), p.status) ? 1 : 0;
          if (okf) p.sk_flags[w.slot * 4 + quarter] = 0u;   // the only waiter resets it for the next launch
        }
        parts_ok = __shfl_sync(0xffffffffu, okf, 0) != 0;
      }
      if (!parts_ok) { *abort_flag = 1; break; }
      // Sum of the other parts' accumulators for one 32-column chunk; issued one chunk ahead so that the loads
      // (L2 latency) overlap the epilogue of the previous chunk.
      float4 pre[8];
      auto load_parts = [&](int c) {
#pragma unroll
        for (int q = 0; q < 8; ++q) pre[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < p.sk_split - 1; ++j) {
          const float4* src = reinterpret_cast<const float4*>(
              p.sk_ws + ((long long)(w.slot * (p.sk_split - 1) + j) * (BLOCK_N / 32) + c) * (kBlockM * 32) +
              (quarter * 32 + lane) * 4);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 v = __ldcg(src + q * kBlockM);
            pre[q].x += v.x; pre[q].y += v.y; pre[q].z += v.z; pre[q].w += v.w;
          }
        }
      };
      if (w.split == 0) load_parts(0);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (w.split == 0) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            r[q * 4 + 0] = __float_as_uint(__uint_as_float(r[q * 4 + 0]) + pre[q].x);
            r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + pre[q].y);
            r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + pre[q].z);
            r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + pre[q].w);
          }
          if (c + 1 < BLOCK_N / 32) load_parts(c + 1);
        }
        const int col0 = n_blk * BLOCK_N + c * 32;
        if (row < p.M && col0 < p.N) epilogue_store_chunk(p, row, col0, r);
      }
      done.fence();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(tempty_bar(buf));
        done(m_blk, n_blk);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // Give copies that are still in flight a bounded chance to land before shared memory is released.
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
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// Host: fill tile counts and pick BLOCK_N when the caller did not.
inline int pick_block_n(int M, int N, int sms) {
  const int mb = (M + kBlockM - 1) / kBlockM;
  auto eff = [&](int bn) {
    const long long tiles = (long long)mb * ((N + bn - 1) / bn);
    const long long waves = (tiles + sms - 1) / sms;
    const double useful = double(M) * double(N);
    const double done = double(waves) * sms * kBlockM * bn;
    return useful / done;
  };
  const double e256 = eff(256), e128 = eff(128) * 0.84;  // measured: the 128-wide tile runs at ~0.84 of the 256-wide one
  return (e256 >= e128) ? 256 : 128;
}

inline void fill_tiles(GemmParams& p, int block_n) {
  p.m_blocks = (p.M + kBlockM - 1) / kBlockM;
  p.n_blocks = (p.N + block_n - 1) / block_n;
  p.k_blocks = (p.K + kBlockK - 1) / kBlockK;
  p.num_tiles = p.m_blocks * p.n_blocks;
  p.group_m = 16;
  p.raster = 0; p.rot = 0; p.k_rot = 0;
  p.dp_tiles = p.num_tiles; p.sk_tiles = 0; p.sk_split = 1;
  p.sk_ws = nullptr; p.sk_flags = nullptr;
}

// How many ways the tiles of the last, partly filled wave are cut along K (1 = not cut) on `grid` CTAs.
inline int tail_split(int num_tiles, int k_blocks, int grid) {
  if (grid <= 0 || num_tiles <= grid) return 1;        // a single wave: nothing to balance against
  const int rem = num_tiles % grid;
  if (rem == 0) return 1;
  // Measured on B200: the cut pays off only when a tile's K loop is long (the tail wave of a short-K GEMM is bound
  // by L2 bandwidth, not by the tensor core, and already runs faster with fewer CTAs) and with few parts per tile.
  if (k_blocks < 64) return 1;
  int s = grid / rem;
  if (s > 4) s = 4;
  return s < 1 ? 1 : s;
}

// Time of a GEMM in units of one full 128 x 256 tile wave, used to pick the tile width.
inline double wave_cost(int M, int N, int K, int sms, int bn) {
  const int tiles = ((M + kBlockM - 1) / kBlockM) * ((N + bn - 1) / bn);
  const int grid = tiles < sms ? tiles : sms;
  const int kb = (K + kBlockK - 1) / kBlockK;
  const int s = tail_split(tiles, kb, grid);
  double waves;
  if (s > 1) waves = double(tiles / grid) + 1.0 / s + 0.06;   // + the workspace round trip of the cut tiles
  else       waves = double((tiles + grid - 1) / grid);
  return waves * (bn == 256 ? 1.0 : 0.5 / 0.84);   // measured: the 128-wide tile runs at ~0.84 of the 256-wide one
}

inline int pick_block_n_split(int M, int N, int K, int sms) {
  return wave_cost(M, N, K, sms, 256) <= wave_cost(M, N, K, sms, 128) ? 256 : 128;
}

// Host: tensor maps for the two operands.
inline int make_operand_maps(CUtensorMap* tmA, CUtensorMap* tmB, const void* A, const void* B, int M, int N, int K,
                             long long lda, long long ldb, int a_major, int b_major, int block_n) {
  int r;
  if (a_major == 0) r = encode_tmap_2d(tmA, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBlockK, kBlockM, 1);
  else              r = encode_tmap_2d(tmA, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, kBlockK, 1);
  if (r) return 1000 + r;
  if (b_major == 0) r = encode_tmap_2d(tmB, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, kBlockK, block_n, 1);
  else              r = encode_tmap_2d(tmB, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, kBlockK, 1);
  if (r) return 2000 + r;
  return 0;
}

}  // namespace lt
