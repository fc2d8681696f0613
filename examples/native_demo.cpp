// A C++ program on the host runtime alone (liblt_host.so, no Python, no CUDA): the pieces a serving or training
// front end written in C++ would use.  It writes and reads back a parameter checkpoint, walks a shuffled data set with
// the prefetching loader, runs a continuous-batching schedule with a stand-in model, evaluates and differentiates a JIT
// expression, and has two threads meet at a barrier of the TCP store.  Built by the top-level CMakeLists.txt
// (target lt_native_demo) or by hand:
//   g++ -std=c++17 -pthread -I csrc/runtime examples/native_demo.cpp -L litetorch_b200/_lib -llt_host -o lt_native_demo
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "lt_host.h"

static int failures = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) { std::printf("FAILED %s:%d  %s\n", __FILE__, __LINE__, #cond); ++failures; } \
  } while (0)

static void checkpoint(const std::string& dir) {
  const std::string path = dir + "/weights.lt";
  std::vector<float> w = {1.5f, -2.0f, 3.25f, 0.5f, 0.0f, 7.0f};
  const int64_t dims[2] = {2, 3};
  void* wr = lt_ckpt_writer_open(path.c_str(), "LTW1");
  EXPECT(wr != nullptr);
  lt_ckpt_write_u32(wr, 1);                                   // one tensor
  lt_ckpt_write_tensor(wr, 2, dims, w.data(), w.size());
  EXPECT(lt_ckpt_writer_close(wr) == 0);                      // the file appears under its name only now

  char magic[4];
  int err = 0;
  void* rd = lt_ckpt_reader_open(path.c_str(), magic, &err);  // the CRC is checked before anything is handed out
  EXPECT(rd != nullptr && std::memcmp(magic, "LTW1", 4) == 0);
  uint32_t count = 0;
  int nd = 0;
  int64_t got_dims[8];
  uint64_t numel = 0;
  std::vector<float> back(6);
  EXPECT(lt_ckpt_read_u32(rd, &count) == 0 && count == 1);
  EXPECT(lt_ckpt_read_tensor_header(rd, &nd, got_dims, &numel) == 0 && nd == 2 && got_dims[1] == 3 && numel == 6);
  EXPECT(lt_ckpt_read_tensor_data(rd, back.data(), numel) == 0 && back == w);
  lt_ckpt_reader_close(rd);
}

static void loader() {
  const uint64_t n = 10;
  std::vector<float> x(n * 2), y(n);
  for (uint64_t i = 0; i < n; ++i) { x[2 * i] = float(i); x[2 * i + 1] = float(i) + 0.5f; y[i] = float(i); }
  void* dl = lt_dl_create(x.data(), y.data(), n, 2, 1, /*batch*/ 4, /*shuffle*/ 1, /*seed*/ 7, /*prefetch*/ 2);
  lt_dl_reset(dl);
  std::vector<float> bx(8), by(4);
  uint64_t count = 0, seen = 0;
  double sum = 0;
  while (lt_dl_next(dl, bx.data(), by.data(), &count) == 1 && count > 0) {
    for (uint64_t i = 0; i < count; ++i) { EXPECT(bx[2 * i] == by[i]); sum += by[i]; }
    seen += count;
  }
  EXPECT(seen == n && sum == 45.0);
  lt_dl_destroy(dl);
}

static void serving() {
  // stand-in model: the next token is the previous one plus one
  void* s = lt_sched_create(/*blocks*/ 10, /*block size*/ 4, /*max seqs*/ 2, /*token budget*/ 8, /*eos*/ -1);
  const int32_t p1[] = {1, 2, 3, 4, 5, 6}, p2[] = {10, 11};
  lt_sched_add_request(s, 1, p1, 6, 4);
  lt_sched_add_request(s, 2, p2, 2, 4);
  int64_t ids[4], done[4];
  int32_t start[4], len[4], toks[64];
  int finished = 0;
  for (int step = 0; step < 50 && finished < 2; ++step) {
    const int n = lt_sched_plan(s, ids, start, len, 4);
    for (int i = 0; i < n; ++i) {
      int prompt_len = 0;
      const int total = lt_sched_tokens(s, ids[i], toks, 64, &prompt_len);
      if (len[i] > 0) {                                       // prefill chunk: a token only once the prompt is complete
        const bool complete = start[i] + len[i] >= prompt_len;
        lt_sched_commit(s, ids[i], complete ? toks[prompt_len - 1] + 1 : -1);
      } else {
        lt_sched_commit(s, ids[i], toks[total - 1] + 1);
      }
    }
    const int k = lt_sched_pop_finished(s, done, 4);
    for (int i = 0; i < k; ++i) {
      int prompt_len = 0;
      const int total = lt_sched_tokens(s, done[i], toks, 64, &prompt_len);
      EXPECT(total == prompt_len + 4 && toks[total - 1] == toks[prompt_len - 1] + 4);
      lt_sched_release(s, done[i]);
    }
    finished += k;
  }
  EXPECT(finished == 2 && lt_sched_num_free_blocks(s) == 10);
  lt_sched_destroy(s);
}

static void jit() {
  const int x = lt_jit_input("x"), y = lt_jit_input("y");
  const int expr = lt_jit_unary(/*RELU*/ 6, lt_jit_binary(/*MUL*/ 4, x, y));
  const int ddx = lt_jit_derivative(expr, "x");
  const float xv[] = {-2, 3, 4, -5}, yv[] = {2, 2, -2, 2};
  const char* names[] = {"x", "y"};
  const float* ptrs[] = {xv, yv};
  float out[4], grad[4];
  EXPECT(lt_jit_eval_cpu(expr, names, ptrs, 2, 4, out) == 0 && out[1] == 6.0f && out[0] == 0.0f);
  EXPECT(lt_jit_eval_cpu(ddx, names, ptrs, 2, 4, grad) == 0 && grad[1] == 2.0f && grad[2] == 0.0f);
}

static void store() {
  int port = 0;
  void* server = lt_store_server_start(0, &port);
  EXPECT(server != nullptr && port > 0);
  auto rank = [port](int r) {
    void* c = lt_store_connect("127.0.0.1", port, 5000);
    if (r == 0) lt_store_set(c, "greeting", "hello", 5);
    char buf[16] = {0};
    EXPECT(lt_store_get(c, "greeting", buf, sizeof(buf), 5000) == 5 && std::strcmp(buf, "hello") == 0);
    EXPECT(lt_store_barrier(c, "ready", 2, 5000) == 0);
    lt_store_close(c);
  };
  std::thread a(rank, 0), b(rank, 1);
  a.join();
  b.join();
  lt_store_server_stop(server);
}

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  checkpoint(dir);
  loader();
  serving();
  jit();
  store();
  std::printf("threads in the host pool: %d\n", lt_pool_threads());
  std::printf(failures == 0 ? "native demo: all checks passed\n" : "native demo: %d checks FAILED\n", failures);
  return failures == 0 ? 0 : 1;
}
