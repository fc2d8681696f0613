// Serving scheduler, prefix cache, data loader, token stream, checkpoint reader / writer and the JIT expression tree of the host
// runtime under sanitizers (built by tests/test_sanitizers_cpu.py with the runtime's sources).  The scheduler and the
// prefix cache are driven from several threads, as a serving front end with one engine thread would; the data loader
// has its own prefetch thread; checkpoints are written, read back, corrupted and truncated.
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* lt_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_num_batched_tokens, int eos_id);
void lt_sched_destroy(void* h);
int lt_sched_add_request(void* h, int64_t id, const int32_t* prompt, int prompt_len, int max_new_tokens);
int lt_sched_plan(void* h, int64_t* req_ids, int32_t* chunk_start, int32_t* chunk_len, int cap);
int lt_sched_commit(void* h, int64_t id, int32_t token);
int lt_sched_tokens(void* h, int64_t id, int32_t* out, int cap, int* prompt_len);
int lt_sched_block_table(void* h, int64_t id, int32_t* out, int cap);
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
void* lt_dl_create(const float* x, const float* y, uint64_t n, uint64_t x_stride, uint64_t y_stride, uint64_t batch,
                   int shuffle, uint64_t seed, int prefetch_limit);
void lt_dl_destroy(void* h);
void lt_dl_reset(void* h);
int lt_dl_next(void* h, float* x_out, float* y_out, uint64_t* count);
int lt_dl_save_state(void* h, const char* path);
int lt_dl_load_state(void* h, const char* path);
void* lt_ckpt_writer_open(const char* path, const char* magic4);
int lt_ckpt_write_u32(void* h, uint32_t v);
int lt_ckpt_write_tensor(void* h, int ndims, const int64_t* dims, const float* data, uint64_t numel);
int lt_ckpt_writer_close(void* h);
void* lt_ckpt_reader_open(const char* path, char* magic_out4, int* err);
int lt_ckpt_read_u32(void* h, uint32_t* v);
int lt_ckpt_read_tensor_header(void* h, int* ndims, int64_t* dims, uint64_t* numel);
int lt_ckpt_read_tensor_data(void* h, float* out, uint64_t numel);
void lt_ckpt_reader_close(void* h);
void* lt_ts_open(const char* path, int token_bytes, uint64_t seq_len, uint64_t batch, int shuffle, uint64_t seed, int rank,
                 int world, int prefetch);
void lt_ts_close(void* h);
uint64_t lt_ts_batches_per_epoch(void* h);
uint64_t lt_ts_epoch(void* h);
uint64_t lt_ts_position(void* h);
int lt_ts_next(void* h, int64_t* tokens_out, int64_t* targets_out);
void lt_ts_next_epoch(void* h);
void lt_ts_seek(void* h, uint64_t epoch, uint64_t position);
int lt_jit_input(const char* name);
int lt_jit_const(float v);
int lt_jit_binary(int op, int a, int b);
int lt_jit_unary(int op, int a);
int lt_jit_derivative(int node, const char* wrt);
int lt_jit_serialize(int node, char* buf, int cap);
int lt_jit_deserialize(const char* text);
int lt_jit_eval_cpu(int node, const char* const* names, const float* const* ptrs, int n_inputs, uint64_t n, float* out);
}

static int failures = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) { std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__); ++failures; } \
  } while (0)

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : ".";
  // ---- scheduler: four client threads submit requests while one engine thread plans and commits
  {
    void* s = lt_sched_create(256, 16, 8, 64, /*eos*/ 2);
    constexpr int kClients = 4, kPerClient = 25;
    std::atomic<int> submitted{0};
    std::vector<std::thread> clients;
    for (int c = 0; c < kClients; ++c)
      clients.emplace_back([&, c] {
        for (int i = 0; i < kPerClient; ++i) {
          std::vector<int32_t> prompt(5 + (i * 7 + c) % 40, 7);
          if (lt_sched_add_request(s, int64_t(c) * 1000 + i, prompt.data(), int(prompt.size()), 1 + i % 6) == 0)
            submitted.fetch_add(1);
        }
      });
    int finished = 0, steps = 0;
    int64_t ids[16];
    int32_t start[16], len[16];
    while (finished < kClients * kPerClient && steps < 100000) {
      ++steps;
      const int n = lt_sched_plan(s, ids, start, len, 16);
      for (int i = 0; i < n; ++i) lt_sched_commit(s, ids[i], 5);
      int64_t done[16];
      const int nd = lt_sched_pop_finished(s, done, 16);
      for (int i = 0; i < nd; ++i) {
        int32_t toks[128];
        int plen = 0;
        const int total = lt_sched_tokens(s, done[i], toks, 128, &plen);
        if (total <= plen) ++failures;
        lt_sched_release(s, done[i]);
      }
      finished += nd;
      if (n == 0 && nd == 0) std::this_thread::yield();
    }
    for (auto& t : clients) t.join();
    CHECK(submitted.load() == kClients * kPerClient);
    CHECK(finished == kClients * kPerClient);
    CHECK(lt_sched_num_running(s) == 0 && lt_sched_num_pending(s) == 0);
    CHECK(lt_sched_num_free_blocks(s) == 256);
    lt_sched_destroy(s);
  }
  // ---- prefix cache: concurrent inserts and lookups with eviction
  {
    void* pc = lt_prefix_create(32);
    std::vector<std::thread> ts;
    std::atomic<int> bad{0};
    for (int t = 0; t < 4; ++t)
      ts.emplace_back([&, t] {
        for (int i = 0; i < 200; ++i) {
          std::vector<int32_t> toks(16 + (i % 4) * 16);
          for (size_t k = 0; k < toks.size(); ++k) toks[k] = int32_t((t * 131 + i * 17 + int(k)) % 1000);
          std::vector<int32_t> blocks(toks.size() / 16, t);
          lt_prefix_insert(pc, toks.data(), int(toks.size()), blocks.data(), int(blocks.size()));
          int32_t out[8];
          int nb = 0;
          const int hit = lt_prefix_lookup(pc, toks.data(), int(toks.size()), 16, out, 8, &nb);
          if (hit < 0 || hit > int(toks.size()) || (hit > 0 && nb != hit / 16)) bad.fetch_add(1);
        }
      });
    for (auto& t : ts) t.join();
    CHECK(bad.load() == 0);
    CHECK(lt_prefix_size(pc) <= 32);
    lt_prefix_destroy(pc);
  }
  // ---- data loader: two epochs with shuffling, state saved in the middle and restored into a second loader
  {
    const uint64_t n = 103, xs = 3, ys = 1, batch = 8;
    std::vector<float> x(n * xs), y(n * ys);
    for (uint64_t i = 0; i < n; ++i) { y[i] = float(i); for (uint64_t k = 0; k < xs; ++k) x[i * xs + k] = float(i) + 0.25f * k; }
    void* dl = lt_dl_create(x.data(), y.data(), n, xs, ys, batch, 1, 1234, 3);
    std::vector<float> bx(batch * xs), by(batch * ys);
    uint64_t count = 0, seen = 0;
    std::vector<int> hits(n, 0);
    const std::string state = dir + "/dl_state.bin";
    int batches = 0;
    while (lt_dl_next(dl, bx.data(), by.data(), &count)) {
      for (uint64_t i = 0; i < count; ++i) { hits[size_t(by[i])]++; CHECK(bx[i * xs] == by[i]); }
      seen += count;
      if (++batches == 5) CHECK(lt_dl_save_state(dl, state.c_str()) == 0);
    }
    CHECK(seen == n);
    for (uint64_t i = 0; i < n; ++i) CHECK(hits[i] == 1);
    lt_dl_reset(dl);
    seen = 0;
    while (lt_dl_next(dl, bx.data(), by.data(), &count)) seen += count;
    CHECK(seen == n);
    void* dl2 = lt_dl_create(x.data(), y.data(), n, xs, ys, batch, 1, 99, 3);
    CHECK(lt_dl_load_state(dl2, state.c_str()) == 0);
    uint64_t rest = 0;
    while (lt_dl_next(dl2, bx.data(), by.data(), &count)) rest += count;
    CHECK(rest == n - 5 * batch);
    lt_dl_destroy(dl2);
    lt_dl_destroy(dl);
  }
  // ---- data loader, batches large enough to be assembled on the thread pool out of pooled host blocks; two loaders at once
  {
    const uint64_t n = 3000, xs = 300, ys = 1, batch = 1024;
    std::vector<float> x(n * xs), y(n * ys);
    for (uint64_t i = 0; i < n; ++i) { y[i] = float(i); for (uint64_t k = 0; k < xs; ++k) x[i * xs + k] = float(i) + float(k) / 1024.f; }
    std::atomic<int> bad{0};
    auto consume = [&](uint64_t seed) {
      void* dl = lt_dl_create(x.data(), y.data(), n, xs, ys, batch, 1, seed, 2);
      std::vector<float> bx(batch * xs), by(batch * ys);
      uint64_t count = 0, seen = 0;
      for (int epoch = 0; epoch < 2; ++epoch) {
        while (lt_dl_next(dl, bx.data(), by.data(), &count)) {
          for (uint64_t i = 0; i < count; ++i)
            if (bx[i * xs] != by[i] || bx[i * xs + xs - 1] != by[i] + float(xs - 1) / 1024.f) bad++;
          seen += count;
        }
        lt_dl_reset(dl);
      }
      if (seen != 2 * n) bad++;
      lt_dl_destroy(dl);
    };
    std::thread other(consume, 7);
    consume(8);
    other.join();
    CHECK(bad.load() == 0);
  }
  // ---- token stream: two ranks read an epoch concurrently, seeks and epoch changes race with the prefetch thread
  {
    const std::string path = dir + "/tokens.bin";
    const uint32_t n = 6000;
    {
      std::vector<uint32_t> toks(n);
      for (uint32_t i = 0; i < n; ++i) toks[i] = i;
      FILE* f = fopen(path.c_str(), "wb");
      CHECK(f != nullptr);
      CHECK(fwrite(toks.data(), 4, n, f) == n);
      fclose(f);
    }
    const uint64_t T = 16, B = 4;
    std::atomic<uint64_t> windows{0};
    auto reader = [&](int rank) {
      void* ts = lt_ts_open(path.c_str(), 4, T, B, 1, 9, rank, 2, 3);
      CHECK(ts != nullptr);
      std::vector<int64_t> tok(B * T), tgt(B * T);
      for (int epoch = 0; epoch < 3; ++epoch) {
        uint64_t got = 0;
        while (lt_ts_next(ts, tok.data(), tgt.data()) == 1) {
          for (uint64_t i = 0; i < B * T; ++i) CHECK(tgt[i] == tok[i] + 1);
          ++got;
        }
        CHECK(got == lt_ts_batches_per_epoch(ts));
        windows += got * B;
        lt_ts_next_epoch(ts);
      }
      // seeks while the worker is filling its queue: the batch after a seek is the one at that position
      std::vector<int64_t> ref(B * T);
      lt_ts_seek(ts, 1, 5);
      CHECK(lt_ts_next(ts, ref.data(), tgt.data()) == 1);
      for (int i = 0; i < 20; ++i) {
        lt_ts_seek(ts, uint64_t(i % 3), uint64_t(i));
        lt_ts_seek(ts, 1, 5);
        CHECK(lt_ts_next(ts, tok.data(), tgt.data()) == 1);
        CHECK(tok == ref && lt_ts_epoch(ts) == 1 && lt_ts_position(ts) == 6);
      }
      lt_ts_close(ts);
    };
    std::thread a(reader, 0), b(reader, 1);
    a.join();
    b.join();
    CHECK(windows.load() == 2 * 3 * (((n - 1) / T / 2) / B) * B);
    CHECK(lt_ts_open((dir + "/missing.bin").c_str(), 4, T, B, 1, 0, 0, 1, 2) == nullptr);
    CHECK(lt_ts_open(path.c_str(), 4, T, B, 1, 0, 2, 2, 2) == nullptr);     // rank outside the world
  }
  // ---- checkpoint: round trip, one flipped byte, truncation
  {
    const std::string path = dir + "/w.ltw";
    void* w = lt_ckpt_writer_open(path.c_str(), "LTW1");
    CHECK(w != nullptr);
    std::vector<float> a(6), b(5);
    for (size_t i = 0; i < a.size(); ++i) a[i] = float(i) * 0.5f;
    for (size_t i = 0; i < b.size(); ++i) b[i] = -float(i);
    const int64_t da[2] = {2, 3}, db[1] = {5};
    lt_ckpt_write_u32(w, 2);
    CHECK(lt_ckpt_write_tensor(w, 2, da, a.data(), 6) == 0);
    CHECK(lt_ckpt_write_tensor(w, 1, db, b.data(), 5) == 0);
    CHECK(lt_ckpt_writer_close(w) == 0);
    char magic[5] = {0};
    int err = 0;
    void* r = lt_ckpt_reader_open(path.c_str(), magic, &err);
    CHECK(r != nullptr && err == 0 && std::string(magic, 4) == "LTW1");
    uint32_t cnt = 0;
    CHECK(lt_ckpt_read_u32(r, &cnt) == 0 && cnt == 2);
    int nd = 0;
    int64_t dims[16];
    uint64_t numel = 0;
    CHECK(lt_ckpt_read_tensor_header(r, &nd, dims, &numel) == 0 && nd == 2 && numel == 6);
    std::vector<float> back(6);
    CHECK(lt_ckpt_read_tensor_data(r, back.data(), 6) == 0 && back[5] == 2.5f);
    CHECK(lt_ckpt_read_tensor_header(r, &nd, dims, &numel) == 0 && nd == 1 && numel == 5);
    lt_ckpt_reader_close(r);
    // flip one payload byte -> CRC mismatch; cut the file -> too short or CRC mismatch, never a crash
    std::vector<unsigned char> bytes;
    {
      FILE* f = std::fopen(path.c_str(), "rb");
      CHECK(f != nullptr);
      int ch;
      while ((ch = std::fgetc(f)) != EOF) bytes.push_back((unsigned char)ch);
      std::fclose(f);
    }
    auto write_file = [&](const std::string& p, size_t len, int flip) {
      FILE* f = std::fopen(p.c_str(), "wb");
      for (size_t i = 0; i < len; ++i) std::fputc(bytes[i] ^ (int(i) == flip ? 0x40 : 0), f);
      std::fclose(f);
    };
    write_file(dir + "/bad.ltw", bytes.size(), 20);
    CHECK(lt_ckpt_reader_open((dir + "/bad.ltw").c_str(), magic, &err) == nullptr && err == 3);
    write_file(dir + "/cut.ltw", bytes.size() / 2, -1);
    CHECK(lt_ckpt_reader_open((dir + "/cut.ltw").c_str(), magic, &err) == nullptr && err != 0);
    write_file(dir + "/tiny.ltw", 5, -1);
    CHECK(lt_ckpt_reader_open((dir + "/tiny.ltw").c_str(), magic, &err) == nullptr && err == 2);
  }
  // ---- JIT tree: f = sigmoid(x * y + 3) ; df/dx ; text round trip ; evaluation
  {
    const int x = lt_jit_input("x"), y = lt_jit_input("y");
    const int f = lt_jit_unary(/*SIGMOID*/ 8, lt_jit_binary(/*ADD*/ 2, lt_jit_binary(/*MUL*/ 4, x, y), lt_jit_const(3.f)));
    const int dfdx = lt_jit_derivative(f, "x");
    CHECK(f >= 0 && dfdx >= 0);
    char text[4096];
    const int len = lt_jit_serialize(dfdx, text, sizeof text);
    CHECK(len > 0 && len < int(sizeof text));
    const int again = lt_jit_deserialize(text);
    CHECK(again >= 0);
    const float xv[4] = {0.f, 0.5f, -1.f, 2.f}, yv[4] = {1.f, -2.f, 0.25f, 3.f};
    const char* names[2] = {"x", "y"};
    const float* ptrs[2] = {xv, yv};
    float o1[4], o2[4];
    CHECK(lt_jit_eval_cpu(dfdx, names, ptrs, 2, 4, o1) == 0);
    CHECK(lt_jit_eval_cpu(again, names, ptrs, 2, 4, o2) == 0);
    for (int i = 0; i < 4; ++i) {
      const float s = 1.f / (1.f + std::exp(-(xv[i] * yv[i] + 3.f)));
      CHECK(std::fabs(o1[i] - s * (1.f - s) * yv[i]) < 1e-5f);
      CHECK(o1[i] == o2[i]);
    }
  }
  std::printf(failures ? "FAILED %d\n" : "OK\n", failures);
  return failures ? 1 : 0;
}
