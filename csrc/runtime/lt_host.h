// Public C interface of liblt_host.so, the CUDA-free host runtime (checkpoint I/O, data loader, serving scheduler, stores,
// allocator bookkeeping, JIT expression trees, thread pool).  Every source file of the runtime includes this header, so a
// definition that drifts from its declaration does not compile.  All functions are thread-safe unless a handle is
// documented otherwise; handles are opaque pointers owned by the caller and released by the matching *_destroy / *_close.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif


// ---- allocator.cpp
// Caching block allocator over caller-supplied raw alloc / free functions (ralloc: void* (*)(void* ctx, uint64_t bytes),
// rfree: void (*)(void* ctx, void* ptr)); stats out6 = {allocated, cached, raw allocations, cache hits, splits, merges}.
// LRU bookkeeping of a residency manager: register returns the ids to evict so that the limit holds; evict_fn may be null.
void* lt_pool_create(void* ralloc, void* rfree, void* ctx, uint64_t max_cached, uint64_t max_block, uint64_t round_to);
void* lt_pool_alloc(void* h, uint64_t bytes);
int lt_pool_free(void* h, void* ptr);
void lt_pool_empty_cache(void* h);
void lt_pool_set_max_cached(void* h, uint64_t bytes);
void lt_pool_stats(void* h, uint64_t* out6);
void lt_pool_destroy(void* h);
void* lt_lru_create(uint64_t limit_bytes, void* evict_fn, void* ctx);
void lt_lru_destroy(void* h);
void lt_lru_set_limit(void* h, uint64_t bytes);
uint64_t lt_lru_used(void* h);
uint64_t lt_lru_evictions(void* h);
int lt_lru_register(void* h, uint64_t id, uint64_t bytes, uint64_t* evicted, int cap);
void lt_lru_unregister(void* h, uint64_t id);
void lt_lru_touch(void* h, uint64_t id);
void lt_lru_pin(void* h, uint64_t id, int in_use);

// ---- dataloader.cpp
// Prefetching batch assembler over row-major host arrays x [n, x_stride] and y [n, y_stride].  lt_dl_next fills the caller's
// buffers and returns 1, or 0 at the end of the epoch; save / load the position as an LTDL record (0 on success).
void* lt_dl_create(const float* x, const float* y, uint64_t n, uint64_t x_stride, uint64_t y_stride, uint64_t batch, int shuffle, uint64_t seed, int prefetch_limit);
void lt_dl_destroy(void* h);
void lt_dl_reset(void* h);
int lt_dl_next(void* h, float* x_out, float* y_out, uint64_t* count);
uint64_t lt_dl_epoch(void* h);
uint64_t lt_dl_position(void* h);
int lt_dl_save_state(void* h, const char* path);
int lt_dl_load_state(void* h, const char* path);

// ---- io.cpp
// Checkpoint records: 4-byte magic, scalars and tensor records {u32 ndims, i64 dims, u64 numel, f32 data}, CRC-32 trailer.
// The writer builds the file under a temporary name and renames it in lt_ckpt_writer_close (0 on success).
// lt_ckpt_reader_open validates the CRC first; err: 1 cannot open, 2 truncated, 3 CRC mismatch.
uint32_t lt_crc32(const void* data, uint64_t n);
void* lt_ckpt_writer_open(const char* path, const char* magic4);
int lt_ckpt_write_u32(void* h, uint32_t v);
int lt_ckpt_write_i32(void* h, int32_t v);
int lt_ckpt_write_u64(void* h, uint64_t v);
int lt_ckpt_write_u8(void* h, uint8_t v);
int lt_ckpt_write_bytes(void* h, const void* d, uint64_t n);
int lt_ckpt_write_tensor(void* h, int ndims, const int64_t* dims, const float* data, uint64_t numel);
int lt_ckpt_writer_close(void* h);
void* lt_ckpt_reader_open(const char* path, char* magic_out4, int* err);
int lt_ckpt_read_u32(void* h, uint32_t* v);
int lt_ckpt_read_i32(void* h, int32_t* v);
int lt_ckpt_read_u64(void* h, uint64_t* v);
int lt_ckpt_read_u8(void* h, uint8_t* v);
int lt_ckpt_read_bytes(void* h, void* d, uint64_t n);
uint64_t lt_ckpt_remaining(void* h);
int lt_ckpt_read_tensor_header(void* h, int* ndims, int64_t* dims, uint64_t* numel);
int lt_ckpt_read_tensor_data(void* h, float* out, uint64_t numel);
void lt_ckpt_reader_close(void* h);

// ---- jit.cpp
// Expression trees (nodes are integer handles), symbolic derivatives, text serialisation, the CPU interpreter and the CUDA
// source generator.  Binary / unary op codes are the values of litetorch_b200.jit.OpType.
int lt_jit_input(const char* name);
int lt_jit_const(float v);
int lt_jit_binary(int op, int a, int b);
int lt_jit_unary(int op, int a);
int lt_jit_derivative(int node, const char* wrt);
int lt_jit_node_op(int node);
float lt_jit_node_val(int node);
int lt_jit_node_left(int node);
int lt_jit_node_right(int node);
int lt_jit_node_name(int node, char* buf, int cap);
int lt_jit_serialize(int node, char* buf, int cap);
int lt_jit_deserialize(const char* text);
int lt_jit_eval_cpu(int node, const char* const* names, const float* const* ptrs, int n_inputs, uint64_t n, float* out);
int lt_jit_cuda_source(int node, const char* const* names, int n_inputs, const char* kernel, int dtype, char* buf, int cap);

// ---- scheduler.cpp
// Continuous-batching scheduler: plan admits pending requests and returns one entry per active request (chunk_len > 0: prefill
// that slice of the prompt; 0: decode one token), commit reports the model's token (-1: none yet).  Prefix trie over token ids.
// Guided decoding: allowed[v] = 1 when vocabulary entry v may follow prefix under the pattern ("digits", "prefix:<text>", "regex:<re>").
void* lt_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_num_batched_tokens, int eos_id);
void lt_sched_destroy(void* h);
int lt_sched_add_request(void* h, int64_t id, const int32_t* prompt, int prompt_len, int max_new_tokens);
int lt_sched_plan(void* h, int64_t* req_ids, int32_t* chunk_start, int32_t* chunk_len, int cap);
int lt_sched_commit(void* h, int64_t id, int32_t token);
int lt_sched_tokens(void* h, int64_t id, int32_t* out, int cap, int* prompt_len);
int lt_sched_block_table(void* h, int64_t id, int32_t* out, int cap);
int lt_sched_context_len(void* h, int64_t id);
int lt_sched_pop_finished(void* h, int64_t* ids, int cap);
void lt_sched_release(void* h, int64_t id);
int lt_sched_num_free_blocks(void* h);
int lt_sched_num_running(void* h);
int lt_sched_num_pending(void* h);
void* lt_prefix_create(int capacity);
void lt_prefix_destroy(void* h);
int lt_prefix_insert(void* h, const int32_t* tokens, int n, const int32_t* blocks, int n_blocks);
int lt_prefix_lookup(void* h, const int32_t* tokens, int n, int granularity, int32_t* blocks, int cap, int* n_blocks);
int lt_prefix_size(void* h);
int lt_guided_mask(const char* pattern_c, const char* prefix_c, const char* vocab_blob, const int64_t* vocab_off, int V, uint8_t* allowed);

// ---- store.cpp
// TCP key-value store (one server thread, blocking clients) and a file store: rendezvous keys, counters, barriers, heartbeats.
// Negative return values are errors (-1 connection lost, -2 timeout).
void* lt_store_server_start(int port, int* port_out);
void lt_store_server_stop(void* h);
void* lt_store_connect(const char* host, int port, int timeout_ms);
void lt_store_close(void* h);
int lt_store_set(void* h, const char* key, const void* val, uint64_t len);
int64_t lt_store_get(void* h, const char* key, void* buf, uint64_t cap, int timeout_ms);
int64_t lt_store_add(void* h, const char* key, int64_t delta);
int lt_store_heartbeat(void* h, int rank);
void lt_store_set_timeout(void* h, int timeout_ms);
int lt_store_alive(void* h);
int lt_store_silent_ranks(void* h, int world, int ttl_ms, int32_t* ranks, int cap);
int lt_store_dead_ranks(void* h, int ttl_ms, int32_t* ranks, int cap);
int lt_store_barrier(void* h, const char* key, int world, int timeout_ms);
int lt_filestore_set(const char* dir, const char* key, const void* val, uint64_t len);
int64_t lt_filestore_get(const char* dir, const char* key, void* buf, uint64_t cap, int timeout_ms);

// ---- threadpool.cpp
// Host thread pool (LITETORCH_NUM_THREADS, default: hardware threads).  fn_ptr: void (*)(void* ctx, uint64_t begin, uint64_t end).
int lt_pool_threads(void);
void lt_parallel_for(void* fn_ptr, void* ctx, uint64_t n, uint64_t min_parallel);

// ---- tokenstream.cpp
// Token-stream loader for language-model training over a memory-mapped file of uint16 / uint32 token ids: windows of
// seq_len + 1 tokens, permuted per epoch from (seed, epoch), dealt to the ranks round-robin, widened to int64 by a
// prefetch thread.  lt_ts_next returns 1 with a batch ([batch, seq_len] inputs and targets) or 0 at the end of the epoch;
// the position is (epoch, batch index): lt_ts_seek resumes exactly.
void* lt_ts_open(const char* path, int token_bytes, uint64_t seq_len, uint64_t batch, int shuffle, uint64_t seed, int rank, int world, int prefetch);
void lt_ts_close(void* h);
uint64_t lt_ts_num_tokens(void* h);
uint64_t lt_ts_num_windows(void* h);
uint64_t lt_ts_batches_per_epoch(void* h);
uint64_t lt_ts_epoch(void* h);
uint64_t lt_ts_position(void* h);
int lt_ts_next(void* h, int64_t* tokens_out, int64_t* targets_out);
void lt_ts_next_epoch(void* h);
void lt_ts_seek(void* h, uint64_t epoch, uint64_t position);

#ifdef __cplusplus
}  // extern "C"
#endif
