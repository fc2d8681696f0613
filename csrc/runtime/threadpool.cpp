// Small fixed thread pool with a blocking parallel_for, used by host-side data preparation and
// checkpoint I/O.  Same contract as the reference pool (include/litetorch/thread_pool.h:15-157): ranges
// shorter than a threshold run inline on the caller, the caller executes the last chunk itself.
#include "lt_host.h"

#include <cstdlib>
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <queue>
#include <thread>
#include <vector>

namespace {

typedef void (*RangeFn)(uint64_t begin, uint64_t end, void* ctx);

struct PoolT {
  std::vector<std::thread> workers;
  std::queue<std::function<void()>> tasks;
  std::mutex mu;
  std::condition_variable cv;
  bool stop = false;
  explicit PoolT(unsigned n) {
    for (unsigned i = 0; i < n; ++i)
      workers.emplace_back([this] {
        for (;;) {
          std::function<void()> t;
          {
            std::unique_lock<std::mutex> lk(mu);
            cv.wait(lk, [this] { return stop || !tasks.empty(); });
            if (stop && tasks.empty()) return;
            t = std::move(tasks.front());
            tasks.pop();
          }
          t();
        }
      });
  }
  ~PoolT() {
    { std::lock_guard<std::mutex> lk(mu); stop = true; }
    cv.notify_all();
    for (auto& w : workers) w.join();
  }
};

PoolT& pool() {
  // LITETORCH_NUM_THREADS (documented by the reference, docs-en/2.installation.md:100) caps the pool; default: every core.
  static PoolT p([] {
    unsigned n = std::max(1u, std::thread::hardware_concurrency());
    if (const char* e = std::getenv("LITETORCH_NUM_THREADS")) {
      const long v = std::strtol(e, nullptr, 10);
      if (v >= 1 && v <= 1024) n = unsigned(v);
    }
    return n;
  }());
  return p;
}

}  // namespace

extern "C" {

int lt_pool_threads() { return int(pool().workers.size()); }

// Calls fn(begin, end, ctx) over [0, n) split into chunks; runs inline when n < min_parallel.
void lt_parallel_for(void* fn_ptr, void* ctx, uint64_t n, uint64_t min_parallel) {
  RangeFn fn = reinterpret_cast<RangeFn>(fn_ptr);
  if (n == 0) return;
  PoolT& p = pool();
  const uint64_t nthreads = p.workers.size() + 1;
  if (n < (min_parallel ? min_parallel : 50000) || nthreads == 1) { fn(0, n, ctx); return; }
  const uint64_t chunk = (n + nthreads - 1) / nthreads;
  // Completion state shared with the tasks: it lives on the heap and every task holds a reference, so a worker that is
  // still inside its notification when the caller wakes up never touches a destroyed mutex (the counter is changed and
  // read under the mutex for the same reason).
  struct Done {
    std::mutex mu;
    std::condition_variable cv;
    uint64_t pending = 0;
  };
  auto done = std::make_shared<Done>();
  uint64_t begin = 0;
  std::vector<std::pair<uint64_t, uint64_t>> ranges;
  while (begin < n) { ranges.push_back({begin, std::min(n, begin + chunk)}); begin += chunk; }
  done->pending = ranges.size() - 1;
  for (size_t i = 0; i + 1 < ranges.size(); ++i) {
    auto r = ranges[i];
    std::lock_guard<std::mutex> lk(p.mu);
    p.tasks.push([=] {
      fn(r.first, r.second, ctx);
      std::lock_guard<std::mutex> lk2(done->mu);
      if (--done->pending == 0) done->cv.notify_all();
    });
  }
  p.cv.notify_all();
  fn(ranges.back().first, ranges.back().second, ctx);
  std::unique_lock<std::mutex> lk(done->mu);
  done->cv.wait(lk, [&] { return done->pending == 0; });
}

}  // extern "C"
