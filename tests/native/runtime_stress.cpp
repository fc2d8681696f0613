// Multi-threaded stress of the host runtime's C ABI, built with -fsanitize=address,undefined or -fsanitize=thread by
// tests/test_sanitizers_cpu.py together with the runtime's own sources.  The reference has no sanitizer builds and one
// 8-thread training stress (tests/stress_test.cpp:171-214); here the pieces that are shared between threads (host
// memory pool, LRU residency list, thread pool, TCP store with heartbeats and barriers) are driven from 8 threads at once.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

extern "C" {
int lt_pool_threads();
void lt_parallel_for(void* fn_ptr, void* ctx, uint64_t n, uint64_t min_parallel);
void* lt_pool_create(void* ralloc, void* rfree, void* ctx, uint64_t max_cached, uint64_t max_block, uint64_t round_to);
void* lt_pool_alloc(void* h, uint64_t bytes);
int lt_pool_free(void* h, void* ptr);
void lt_pool_empty_cache(void* h);
void lt_pool_stats(void* h, uint64_t* out6);
void lt_pool_destroy(void* h);
void* lt_lru_create(uint64_t limit_bytes, void* evict_fn, void* ctx);
void lt_lru_destroy(void* h);
uint64_t lt_lru_used(void* h);
uint64_t lt_lru_evictions(void* h);
int lt_lru_register(void* h, uint64_t id, uint64_t bytes, uint64_t* evicted, int cap);
void lt_lru_unregister(void* h, uint64_t id);
void lt_lru_touch(void* h, uint64_t id);
void lt_lru_pin(void* h, uint64_t id, int in_use);
void* lt_store_server_start(int port, int* port_out);
void lt_store_server_stop(void* h);
void* lt_store_connect(const char* host, int port, int timeout_ms);
void lt_store_close(void* h);
int lt_store_set(void* h, const char* key, const void* val, uint64_t len);
int64_t lt_store_get(void* h, const char* key, void* buf, uint64_t cap, int timeout_ms);
int64_t lt_store_add(void* h, const char* key, int64_t delta);
int lt_store_heartbeat(void* h, int rank);
int lt_store_dead_ranks(void* h, int ttl_ms, int32_t* ranks, int cap);
int lt_store_barrier(void* h, const char* key, int world, int timeout_ms);
}

static int failures = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) { std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #cond, __LINE__); ++failures; } \
  } while (0)

static std::atomic<uint64_t> g_evicted{0};
static void on_evict(uint64_t, void*) { g_evicted.fetch_add(1); }

static void sum_range(uint64_t b, uint64_t e, void* ctx) {
  auto* acc = static_cast<std::atomic<uint64_t>*>(ctx);
  uint64_t s = 0;
  for (uint64_t i = b; i < e; ++i) s += i;
  acc->fetch_add(s);
}

int main() {
  constexpr int kThreads = 8;
  // ---- thread pool: concurrent parallel_for calls from several callers
  {
    std::vector<std::thread> ts;
    std::atomic<int> bad{0};
    for (int t = 0; t < 4; ++t)
      ts.emplace_back([&] {
        for (int rep = 0; rep < 20; ++rep) {
          std::atomic<uint64_t> acc{0};
          const uint64_t n = 200000;
          lt_parallel_for(reinterpret_cast<void*>(&sum_range), &acc, n, 1000);
          if (acc.load() != n * (n - 1) / 2) bad.fetch_add(1);
        }
      });
    for (auto& t : ts) t.join();
    CHECK(bad.load() == 0);
    CHECK(lt_pool_threads() >= 0);
  }
  // ---- host memory pool: allocate, write, free from 8 threads; blocks are reused and never handed out twice
  {
    void* pool = lt_pool_create(nullptr, nullptr, nullptr, 8u << 20, 1u << 20, 256);
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < kThreads; ++t)
      ts.emplace_back([&, t] {
        std::vector<void*> held;
        for (int i = 0; i < 400; ++i) {
          const uint64_t bytes = 64 + uint64_t((i * 37 + t * 101) % 5000);
          auto* p = static_cast<unsigned char*>(lt_pool_alloc(pool, bytes));
          if (!p) { bad.fetch_add(1); continue; }
          std::memset(p, t + 1, bytes);
          held.push_back(p);
          if (held.size() > 16) {
            auto* q = static_cast<unsigned char*>(held.front());
            if (q[0] != t + 1) bad.fetch_add(1);      // somebody else wrote into a block this thread still owns
            if (lt_pool_free(pool, q) != 0) bad.fetch_add(1);
            held.erase(held.begin());
          }
        }
        for (void* p : held) lt_pool_free(pool, p);
      });
    for (auto& t : ts) t.join();
    CHECK(bad.load() == 0);
    uint64_t st[6];
    lt_pool_stats(pool, st);
    lt_pool_empty_cache(pool);
    lt_pool_destroy(pool);
  }
  // ---- LRU residency list: register / touch / pin / unregister under a tight limit
  {
    void* lru = lt_lru_create(64 * 1024, reinterpret_cast<void*>(&on_evict), nullptr);
    std::vector<std::thread> ts;
    for (int t = 0; t < kThreads; ++t)
      ts.emplace_back([&, t] {
        uint64_t ev[8];
        for (uint64_t i = 0; i < 300; ++i) {
          const uint64_t id = uint64_t(t) * 100000 + i;
          lt_lru_register(lru, id, 4096, ev, 8);
          lt_lru_pin(lru, id, 1);
          lt_lru_touch(lru, id);
          lt_lru_pin(lru, id, 0);
          if (i % 3 == 0) lt_lru_unregister(lru, id);
        }
      });
    for (auto& t : ts) t.join();
    CHECK(lt_lru_used(lru) <= 64 * 1024 + uint64_t(kThreads) * 4096);
    CHECK(lt_lru_evictions(lru) == g_evicted.load());
    CHECK(g_evicted.load() > 0);
    lt_lru_destroy(lru);
  }
  // ---- TCP store: counters, keys, heartbeats and a barrier from 8 client threads against one server
  {
    int port = 0;
    void* srv = lt_store_server_start(0, &port);
    CHECK(srv != nullptr && port > 0);
    std::atomic<int> bad{0};
    std::vector<std::thread> ts;
    for (int t = 0; t < kThreads; ++t)
      ts.emplace_back([&, t] {
        void* c = lt_store_connect("127.0.0.1", port, 5000);
        if (!c) { bad.fetch_add(1); return; }
        char key[32], val[32], buf[64];
        for (int i = 0; i < 50; ++i) {
          lt_store_add(c, "ctr", 1);
          std::snprintf(key, sizeof key, "k%d_%d", t, i);
          std::snprintf(val, sizeof val, "v%d_%d", t, i);
          if (lt_store_set(c, key, val, std::strlen(val)) != 0) bad.fetch_add(1);
          const int64_t n = lt_store_get(c, key, buf, sizeof buf, 2000);
          if (n != int64_t(std::strlen(val)) || std::memcmp(buf, val, size_t(n)) != 0) bad.fetch_add(1);
          lt_store_heartbeat(c, t);
        }
        if (lt_store_barrier(c, "b0", kThreads, 10000) != 0) bad.fetch_add(1);
        lt_store_close(c);
      });
    for (auto& t : ts) t.join();
    void* c = lt_store_connect("127.0.0.1", port, 5000);
    CHECK(c != nullptr);
    CHECK(lt_store_add(c, "ctr", 0) == kThreads * 50);
    int32_t dead[16];
    CHECK(lt_store_dead_ranks(c, 60000, dead, 16) == 0);      // everybody reported within the last minute
    lt_store_close(c);
    lt_store_server_stop(srv);
    CHECK(bad.load() == 0);
  }
  std::printf(failures ? "FAILED %d\n" : "OK\n", failures);
  return failures ? 1 : 0;
}
