// Public C interface of liblt_cuda.so: every sm_100a kernel launcher and the CUDA-side runtime.  Pointers are device
// pointers unless a name says otherwise, `stream` is a cudaStream_t passed as void* (0 = default stream), launchers return
// 0 or a CUDA error code.  Every source file of the library includes this header, so a definition that drifts from its
// declaration does not compile.
#pragma once
#include <stdint.h>
#include <sys/types.h>

struct CUstream_st;
typedef struct CUstream_st* cudaStream_t;

// Description of the next gather-GEMM of a sequence, for prefetching by lt_ag_gemm_bf16 (all fields as in its arguments).
typedef struct LtNextGather {
  int gather_operand, M, N, K, rows_per_rank, pad;
  const void* shard_ptrs[8];
  void* full;
  void* flags;
  unsigned epoch, pad2;
} LtNextGather;

#ifdef __cplusplus
extern "C" {
#endif

// ---- flash_bwd.cu: FlashAttention backward: dQ, dK, dV from dO, O, LSE
void lt_flash_bwd_set_trace(void* buf);
int lt_flash_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                 void* dq, void* dk, void* dv, float* delta, float* dq_acc, int B, int Tq, int Tk, int Hq, int Hkv,
                 int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t, long long sv_b, long long sv_t,
                 long long so_b, long long so_t, long long sdo_b, long long sdo_t, long long sdq_b, long long sdq_t,
                 long long sdk_b, long long sdk_t, float scale, int causal, void* stream);
int lt_flash_bwd_cp(int phase, const void* const* q_ptrs, const void* k, const void* v, const void* o,
                    const void* const* do_ptrs, const float* const* lse_ptrs, const float* const* delta_ptrs,
                    float* const* dq_acc_ptrs, void* dq, void* dk, void* dv, int B, int Tq, int Tk, int Hq, int Hkv,
                    int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t, long long sv_b,
                    long long sv_t, long long so_b, long long so_t, long long sdo_b, long long sdo_t, long long sdq_b,
                    long long sdq_t, long long sdk_b, long long sdk_t, float scale, int causal, int cp_world,
                    int cp_rank, int zigzag, void* stream);

// ---- flash_fwd.cu: FlashAttention forward (tcgen05, S and O in tensor memory): q [B, Tq, Hq, D], k / v [B, Tk, Hkv, D] bf16, D 64 or 128;
// the _cp form takes one K / V tensor per rank (context parallelism)
void lt_flash_fwd_set_trace(void* buf);
int lt_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq, int Tk, int Hq,
                 int Hkv, int D, long long sq_b, long long sq_t, long long sk_b, long long sk_t, long long sv_b,
                 long long sv_t, long long so_b, long long so_t, float scale, int causal, void* stream);
int lt_flash_fwd_cp(const void* q, const void* const* k_ptrs, const void* const* v_ptrs, void* o, float* lse, int B,
                    int Tq, int Tk, int Hq, int Hkv, int D, long long sq_b, long long sq_t, long long sk_b,
                    long long sk_t, long long sv_b, long long sv_t, long long so_b, long long so_t, float scale,
                    int causal, int cp_world, int cp_rank, int zigzag, void* stream);

// ---- fsdp_fused.cu: ZeRO-3 fused paths: all-gather -> GEMM, reduce-scatter -> AdamW, shard gathers, flag barrier between ranks
int lt_ag_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                    long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                    long long ldr, int act, int accumulate, float alpha, int gather_operand,
                    const void* const* shard_ptrs, int world, int rank, int rows_per_rank, void* full, void* flags,
                    unsigned epoch, int n_comm, const LtNextGather* next, void* progress, unsigned progress_base,
                    void* stream);
int lt_gemm_num_tiles(int M, int N, int n_comm);
int lt_rs_adamw(const void* const* grad_ptrs, const void* mc_grads, float* master, float* m, float* v,
                void* param_shard, const long long* segs, int n_seg, float lr, float beta1, float beta2, float eps,
                float wd, float bc1, float bc2, void* my_flags, const void* const* peer_flags, int slot,
                unsigned epoch, int world, int rank, int max_ctas, void* stream);
int lt_gather_shards(const void* const* shard_ptrs, int world, const long long* segs, const void* const* dst_ptrs,
                     int n_seg, int max_ctas, void* stream);
int lt_embedding_fwd_sharded(const long long* idx, const void* const* table_ptrs, void* out, long long n_tok, int D,
                             int V, int rows_per_rank, int world, void* stream);
int lt_signal_barrier(void* my_flags, const void* const* peer_flags, int slot, unsigned epoch, int world, int rank,
                      void* stream);

// ---- gemm_fp8_pair_sm100.cu: block-scaled e4m3 GEMM on CTA pairs
int lt_gemm_fp8_block_pair(const void* A8, const void* B8, void* C, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, const void* a_scale, const void* b_scale, int out_fp32, const void* bias,
                           void* stream);

// ---- gemm_fp8_sm100.cu: block-scaled e4m3 GEMM (1x128 activation scales, 128x128 weight scales, two-level accumulation) and its activation quantiser
int lt_gemm_fp8_block(const void* A8, const void* B8, void* C, int M, int N, int K, long long lda, long long ldb,
                      long long ldc, const void* a_scale, const void* b_scale, int out_fp32, const void* bias,
                      int max_ctas, void* stream);
int lt_quant_fp8_1x128(const void* x, long long ldx, void* q, long long ldq, void* scale_t, int M, int K, void* stream);

// ---- gemm_skinny.cu: weight-streaming GEMM for 9-128 rows
int lt_gemm_skinny_set_target(int ctas_per_sm, int min_chunks_per_warp);
int lt_gemm_skinny_bf16(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy,
                        const void* residual, long long ldr, int M, int N, int K, void* stream);

// ---- gemm_sm100.cu: persistent tcgen05 GEMM: C = epilogue(alpha * op(A) op(B)); a_major / b_major 0 = K contiguous; act 1 = GELU;
// pitches in elements; returns 0, a cudaError_t, or 1000 + CUresult of a failed tensor-map encoding
void lt_gemm_set_pair_mode(int mode);
void lt_gemm_set_tail_split(int enable);
int lt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                 long long ldr, int act, int accumulate, float alpha, int block_n, int max_ctas, void* stream);
int lt_gemm_typed(int kind, const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                  long long ldc, int a_major, int b_major, int out_fp32, const void* bias, const void* residual,
                  long long ldr, int act, int accumulate, float alpha, void* stream);
int lt_gemm_e4m3(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                 long long ldc, int out_fp32, const float* a_scale, const float* b_scale, const void* bias,
                 const void* residual, long long ldr, int act, float alpha, void* stream);

// ---- gemv.cu: GEMV for 1-8 rows
int lt_gemv_bf16(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy,
                 const void* residual, long long ldr, int M, int N, int K, void* stream);

// ---- loss_optim.cu: fused cross-entropy (statistics, then loss and gradient in place), Adam / AdamW / SGD / RMSprop steps, gradient norm and clipping
int lt_ce_stats(const void* logits, long long ldl, const long long* targets, int vocab_start, int N, int V,
                float* stats, void* stream);
int lt_ce_finish(void* logits, long long ldl, const long long* targets, int vocab_start, int N, int V,
                 const float* gstats, float* loss, float grad_scale, long long ignore_index, int write_grad,
                 void* stream);
int lt_adam_flat(float* master, const void* grad, int grad_is_bf16, float* m, float* v, void* param_bf16, long long n,
                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, int adamw,
                 const float* dyn, void* stream);
int lt_adam_table(const void* p_ptrs, const void* g_ptrs, const void* m_ptrs, const void* v_ptrs, const void* p16_ptrs,
                  const long long* numel, const int* g_is_bf16, const int* chunk_tensor, const long long* chunk_off,
                  int n_chunks, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                  int adamw, const float* dyn, void* stream);
int lt_adam_chunk_elems(void);
int lt_adam_q8(void* p, int p_bf16, const void* g, int g_bf16, void* mq, void* vq, long long n, float lr, float beta1,
               float beta2, float eps, float wd, float bc1, float bc2, int fp8, int first, const float* scale_old,
               float* scale_new, void* amax, float* hist, int* hist_n, void* stream);
int lt_sgd_flat(float* p, const float* g, float* vel, long long n, float lr, float momentum, float wd, void* stream);
int lt_rmsprop_flat(float* p, const float* g, float* sq, long long n, float lr, float alpha, float eps, float wd,
                    void* stream);
int lt_sumsq(const void* x, int is_bf16, long long n, float* out, void* stream);
int lt_clip_coef(const float* stats, float* dyn, float max_norm, float inv_scale, void* stream);

// ---- misc.cu: router, dropout, softmax, quantisers, reductions, strided copy, GradScaler unscale-and-check
int lt_moe_router(const void* logits, int dtype, float* probs, float* topk_w, int* topk_idx, int* counts, float* mass,
                  int N, int E, int k, int renorm, void* stream);
int lt_moe_router_bwd(const float* probs, const int* topk_idx, const float* topk_w, const float* d_topk_w,
                      const float* d_probs, float* dlogits, int N, int E, int k, int renorm, void* stream);
int lt_dropout(const void* x, void* y, long long n, int dtype, float p, unsigned long long seed,
               unsigned long long offset, void* stream);
int lt_softmax_fwd(const void* x, void* y, long long rows, int D, int dtype, void* stream);
int lt_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int D, int dtype, void* stream);
int lt_quant_fp8_128x128(const void* w, long long ldw, void* q, long long ldq, float* scales, int N, int K,
                         void* stream);
int lt_unscale_check(void* g, long long n, int dtype, float inv_scale, int* found_inf, void* stream);
int lt_reduce_parts(void);
int lt_reduce_all(const void* x, long long n, int dtype, int mode, float* part, float* out, void* stream);
int lt_strided_copy(const void* src, void* dst, int ndim, const long long* shape, const long long* src_stride,
                    const long long* dst_stride, int elem_bytes, void* stream);
int lt_moe_expert_bwd(const void* gu, const void* dh_u, const void* w, const void* slot_src, void* dgu, void* hw,
                      void* dw, int S, int F, void* stream);
int lt_quant_e4m3_rows(const void* x, long long ldx, void* q, long long ldq, float* scale, int rows, int cols,
                       void* stream);
int lt_quant_int8_tensor(const void* x, int is_bf16, void* q, long long n, float scale, void* stream);
int lt_quant_int8_rows(const void* x, int is_bf16, void* q, float* scale, int rows, int cols, void* stream);

// ---- moe_fused.cu: MoE dispatch fused into the first grouped GEMM, combine fused into the second one's epilogue
int lt_moe_gather_gemm(const void* const* src_ptrs, int world, const void* slot_src, const int* group_of_mblk,
                       int slots, const void* B, int n_experts, int N, int K, int b_major, void* slot_buf, void* flags,
                       unsigned epoch, void* C, const float* row_scale, int n_comm, void* stream);
int lt_moe_gemm_scatter(const void* A, const int* group_of_mblk, int slots, const void* B, int n_experts, int N, int K,
                        int b_major, const void* slot_dst, const float* row_weight, const void* const* acc_ptrs,
                        int world, void* stream);

// ---- norm.cu: RMSNorm / LayerNorm forward and backward (optional residual add)
int lt_norm_bwd_ctas(int M);
int lt_norm_fwd(int layer_norm, const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out,
                float* mean_out, float* rstd_out, int M, int D, float eps, void* stream);
int lt_norm_bwd(int layer_norm, const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                const void* dres, void* dx, float* dw_part, float* db_part, void* dw, void* db, int grads_fp32,
                int accumulate, int M, int D, void* stream);
int lt_norm_bwd_noalloc(int layer_norm, const void* dy, const void* x, const void* w, const float* mean,
                        const float* rstd, const void* dres, void* dx, void* dw, void* db, int grads_fp32,
                        int accumulate, int M, int D, void* stream);

// ---- paged_decode.cu: decode attention over a block-paged KV cache, cache append
int lt_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                    const int* context_lens, float* part, void* o, int S, int Hq, int Hkv, int D, int block_size,
                    int max_blocks, int num_blocks, int splits, float scale, int kv_fp8, float k_scale, float v_scale,
                    void* stream);
int lt_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int* slots, long long n_tok,
                 int Hkv, int D, int block_size, int kv_fp8, float k_scale, float v_scale, void* stream);

// ---- pointwise.cu: RoPE, SwiGLU, GELU, embedding, casts, axpby
int lt_rope(void* x, const float* cos_t, const float* sin_t, const int* pos, long long rows, int T, int heads, int hd,
            long long row_stride, int backward, void* stream);
int lt_swiglu_fwd(const void* gu, void* h, long long M, int F, void* stream);
int lt_swiglu_bwd(const void* gu, const void* dh, void* dgu, long long M, int F, void* stream);
int lt_gelu_fwd(const void* x, void* y, long long n, void* stream);
int lt_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream);
int lt_axpby(const void* a, const void* b, void* out, float alpha, float beta, long long n, void* stream);
int lt_embedding_fwd(const long long* idx, const void* table, void* out, long long n_tok, int D, int V, void* stream);
int lt_embedding_bwd(const long long* idx, const void* dout, void* dtable, long long n_tok, int D, int V, void* stream);
int lt_cast_f32_to_bf16(const float* in, void* out, long long n, void* stream);
int lt_cast_bf16_to_f32(const void* in, float* out, long long n, void* stream);

// ---- tp_fused.cu: GEMM with a reduce-scatter epilogue (tensor parallelism)
int lt_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int b_major,
                    const void* const* stage_ptrs, const void* const* counter_ptrs, unsigned epoch, int world,
                    int rank, int rows_per_rank, void* out, long long ldo, const void* bias, const void* residual,
                    long long ldr, void* stream);

// ---- host.cu: per-device status word of the bounded waits, wait budgets
int lt_status_fetch(void);
int lt_sm_count(void);
int lt_set_wait_budget_cycles(long long local_cycles, long long peer_cycles);

// ---- nccl_bridge.cu: NCCL through dlopen(libnccl.so.2): communicator from a 128-byte unique id, collectives and point-to-point on a stream
int lt_nccl_version(void);
int lt_nccl_unique_id(void* out128);
void* lt_nccl_init(const void* id128, int world, int rank, int* err);
int lt_nccl_destroy(void* comm);
int lt_nccl_all_reduce(void* comm, const void* send, void* recv, unsigned long long count, int dtype, int op,
                       void* stream);
int lt_nccl_all_gather(void* comm, const void* send, void* recv, unsigned long long send_count, int dtype,
                       void* stream);
int lt_nccl_reduce_scatter(void* comm, const void* send, void* recv, unsigned long long recv_count, int dtype, int op,
                           void* stream);
int lt_nccl_broadcast(void* comm, const void* send, void* recv, unsigned long long count, int dtype, int root,
                      void* stream);
int lt_nccl_send(void* comm, const void* buf, unsigned long long count, int dtype, int peer, void* stream);
int lt_nccl_recv(void* comm, void* buf, unsigned long long count, int dtype, int peer, void* stream);
int lt_nccl_group_start(void);
int lt_nccl_group_end(void);

// ---- runtime.cu: caching device allocator (PyTorch pluggable-allocator signature), CUDA graph capture / replay, CUDA-IPC symmetric heap, NVRTC compile and launch
void* lt_cuda_alloc(ssize_t size, int device, cudaStream_t stream);
void lt_cuda_free(void* ptr, ssize_t, int device, cudaStream_t stream);
void lt_cuda_record_stream(void* ptr, cudaStream_t stream);
void lt_cuda_empty_cache(void);
void lt_cuda_set_max_cached(uint64_t bytes);
void lt_cuda_alloc_stats(uint64_t* out5);
int lt_ipc_export(void* ptr, void* handle_out, unsigned long long* offset_out);
void* lt_ipc_open(const void* handle, unsigned long long offset, void** base_out, int* err);
int lt_ipc_close(void* base);
int lt_graph_begin_capture(void* stream);
void* lt_graph_end_capture(void* stream, int* err);
int lt_graph_launch(void* exec, void* stream);
void lt_graph_destroy(void* exec);
int lt_jit_compile(const char* source, const char* kernel_name, int n_inputs);
int lt_jit_last_log(char* buf, int cap);
int lt_jit_launch(int handle, const void* const* inputs, int n_inputs, void* out, long long n, void* stream);

#ifdef __cplusplus
}  // extern "C"
#endif
