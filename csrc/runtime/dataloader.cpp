// Prefetching data loader over an in-memory (features, labels) dataset.
//
// Behaviour follows the reference loader (src/data/dataloader.cpp:41-349): one prefetch thread fills a
// bounded queue of batches, a generation counter drops batches that were assembled before a reset or a
// state load, an epoch ends with a short (or empty) batch, and the position can be saved to / restored
// from an `LTDL` file: magic, u64 current_index, u64 worker_index, u64 epoch_id, u8 shuffle, u64 n,
// u64 indices[n], CRC-32 of all preceding bytes.  Batches are assembled straight into buffers the caller
// provides (pinned host memory, so that the copy to the GPU can be asynchronous).
#include "lt_host.h"

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

namespace {

// Batch storage comes from the host block pool shared by all loaders: a prefetch thread allocates and the consumer
// frees a few multi-megabyte blocks per step, which the pool turns into reuse of the same blocks.
void* batch_pool() {
  static void* pool = lt_pool_create(nullptr, nullptr, nullptr, 1ull << 30, 0, 4096);
  return pool;
}

struct PoolBuf {
  float* ptr = nullptr;
  uint64_t n = 0;
  PoolBuf() = default;
  PoolBuf(const PoolBuf&) = delete;
  PoolBuf& operator=(const PoolBuf&) = delete;
  PoolBuf(PoolBuf&& o) noexcept : ptr(o.ptr), n(o.n) { o.ptr = nullptr; o.n = 0; }
  PoolBuf& operator=(PoolBuf&& o) noexcept {
    if (this != &o) { reset(); ptr = o.ptr; n = o.n; o.ptr = nullptr; o.n = 0; }
    return *this;
  }
  ~PoolBuf() { reset(); }
  void reset() {
    if (ptr) lt_pool_free(batch_pool(), ptr);
    ptr = nullptr; n = 0;
  }
  void resize(uint64_t count) {
    reset();
    ptr = static_cast<float*>(lt_pool_alloc(batch_pool(), count * sizeof(float)));
    n = ptr ? count : 0;
  }
  float* data() { return ptr; }
  const float* data() const { return ptr; }
  uint64_t size() const { return n; }
};

struct Batch {
  PoolBuf x, y;
  uint64_t count = 0;
  uint64_t generation = 0;
  uint64_t next_index = 0;  // dataset position after this batch
  bool end_of_epoch = false;
};

struct Loader {
  const float* x;
  const float* y;
  uint64_t n, xs, ys, batch;
  bool shuffle;
  uint64_t seed;
  size_t prefetch_limit;
  std::vector<uint64_t> indices;
  uint64_t current_index = 0;  // consumer position
  uint64_t worker_index = 0;   // producer position
  uint64_t epoch_id = 0;
  uint64_t generation = 0;
  bool worker_done = false;    // producer reached the end of the epoch
  bool stop = false;
  std::deque<Batch> queue;
  std::mutex mu;
  std::condition_variable cv;
  std::thread worker;

  void make_indices() {
    indices.resize(n);
    for (uint64_t i = 0; i < n; ++i) indices[i] = i;
    if (shuffle) {
      std::mt19937_64 rng(seed + epoch_id * 0x9E3779B97F4A7C15ull);
      std::shuffle(indices.begin(), indices.end(), rng);
    }
  }

  struct CopyJob {
    const Loader* self;
    Batch* out;
    const uint64_t* idx;
  };
  static void copy_range(uint64_t begin, uint64_t end, void* ctx) {
    const CopyJob& j = *static_cast<const CopyJob*>(ctx);
    const Loader* d = j.self;
    for (uint64_t i = begin; i < end; ++i) {
      memcpy(j.out->x.data() + i * d->xs, d->x + j.idx[i] * d->xs, d->xs * sizeof(float));
      memcpy(j.out->y.data() + i * d->ys, d->y + j.idx[i] * d->ys, d->ys * sizeof(float));
    }
  }

  void run() {
    std::unique_lock<std::mutex> lk(mu);
    while (!stop) {
      cv.wait(lk, [&] { return stop || (!worker_done && queue.size() < prefetch_limit); });
      if (stop) break;
      const uint64_t gen = generation;
      const uint64_t start = worker_index;
      if (start >= n) {
        worker_done = true;
        Batch b;
        b.generation = gen;
        b.end_of_epoch = true;
        b.next_index = n;
        queue.push_back(std::move(b));
        cv.notify_all();
        continue;
      }
      const uint64_t cnt = std::min(batch, n - start);
      std::vector<uint64_t> idx(indices.begin() + start, indices.begin() + start + cnt);
      lk.unlock();
      Batch b;
      b.x.resize(cnt * xs);
      b.y.resize(cnt * ys);
      // Sample rows are copied by the host thread pool once a batch is worth splitting (about 1 MB and up).
      CopyJob job{this, &b, idx.data()};
      const uint64_t floats_per_sample = xs + ys ? xs + ys : 1;
      lt_parallel_for(reinterpret_cast<void*>(&Loader::copy_range), &job, cnt, std::max<uint64_t>(2, (1u << 18) / floats_per_sample));
      b.count = cnt;
      b.generation = gen;
      b.next_index = start + cnt;
      lk.lock();
      if (gen == generation) {  // otherwise a reset happened while the batch was assembled: drop it
        worker_index = start + cnt;
        queue.push_back(std::move(b));
        cv.notify_all();
      }
    }
  }
};

}  // namespace

extern "C" {

void* lt_dl_create(const float* x, const float* y, uint64_t n, uint64_t x_stride, uint64_t y_stride, uint64_t batch,
                   int shuffle, uint64_t seed, int prefetch_limit) {
  Loader* d = new Loader();
  d->x = x; d->y = y; d->n = n; d->xs = x_stride; d->ys = y_stride;
  d->batch = batch ? batch : 1;
  d->shuffle = shuffle != 0;
  d->seed = seed;
  d->prefetch_limit = prefetch_limit > 0 ? size_t(prefetch_limit) : 2;
  d->make_indices();
  d->worker = std::thread([d] { d->run(); });
  return d;
}

void lt_dl_destroy(void* h) {
  Loader* d = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> lk(d->mu);
    d->stop = true;
  }
  d->cv.notify_all();
  if (d->worker.joinable()) d->worker.join();
  delete d;
}

// Starts the next epoch (reshuffles when shuffling is on).
void lt_dl_reset(void* h) {
  Loader* d = static_cast<Loader*>(h);
  std::lock_guard<std::mutex> lk(d->mu);
  d->generation++;
  d->epoch_id++;
  d->queue.clear();
  d->current_index = 0;
  d->worker_index = 0;
  d->worker_done = false;
  d->make_indices();
  d->cv.notify_all();
}

// Copies the next batch into x_out / y_out (room for batch * stride floats). Returns 1 and sets *count,
// or 0 at the end of the epoch.
int lt_dl_next(void* h, float* x_out, float* y_out, uint64_t* count) {
  Loader* d = static_cast<Loader*>(h);
  std::unique_lock<std::mutex> lk(d->mu);
  for (;;) {
    d->cv.wait(lk, [&] { return !d->queue.empty() || d->stop; });
    if (d->stop) return 0;
    Batch b = std::move(d->queue.front());
    d->queue.pop_front();
    d->cv.notify_all();
    if (b.generation != d->generation) continue;  // stale
    if (b.end_of_epoch) {
      // leave a marker so that repeated calls keep answering "end of epoch" until reset
      d->queue.push_front(std::move(b));
      *count = 0;
      return 0;
    }
    memcpy(x_out, b.x.data(), b.x.size() * sizeof(float));
    memcpy(y_out, b.y.data(), b.y.size() * sizeof(float));
    *count = b.count;
    d->current_index = b.next_index;
    return 1;
  }
}

uint64_t lt_dl_epoch(void* h) { return static_cast<Loader*>(h)->epoch_id; }
uint64_t lt_dl_position(void* h) { return static_cast<Loader*>(h)->current_index; }

int lt_dl_save_state(void* h, const char* path) {
  Loader* d = static_cast<Loader*>(h);
  std::lock_guard<std::mutex> lk(d->mu);
  std::vector<uint8_t> buf;
  auto put = [&](const void* p, size_t n) { const uint8_t* b = static_cast<const uint8_t*>(p); buf.insert(buf.end(), b, b + n); };
  put("LTDL", 4);
  const uint64_t cur = d->current_index, wrk = d->current_index, ep = d->epoch_id, cnt = d->indices.size();
  const uint8_t sh = d->shuffle ? 1 : 0;
  put(&cur, 8); put(&wrk, 8); put(&ep, 8); put(&sh, 1); put(&cnt, 8);
  put(d->indices.data(), cnt * 8);
  const uint32_t crc = lt_crc32(buf.data(), buf.size());
  put(&crc, 4);
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  const bool ok = fwrite(buf.data(), 1, buf.size(), f) == buf.size();
  const bool closed = fclose(f) == 0;
  return ok && closed ? 0 : -2;
}

// Returns 0, -1 cannot open, -2 malformed, -3 CRC mismatch, -4 dataset size differs.
int lt_dl_load_state(void* h, const char* path) {
  Loader* d = static_cast<Loader*>(h);
  FILE* f = fopen(path, "rb");
  if (!f) return -1;
  std::vector<uint8_t> buf;
  uint8_t tmp[65536];
  size_t got;
  while ((got = fread(tmp, 1, sizeof(tmp), f)) > 0) buf.insert(buf.end(), tmp, tmp + got);
  fclose(f);
  if (buf.size() < 4 + 8 * 3 + 1 + 8 + 4 || memcmp(buf.data(), "LTDL", 4) != 0) return -2;
  uint32_t stored;
  memcpy(&stored, buf.data() + buf.size() - 4, 4);
  if (stored != lt_crc32(buf.data(), buf.size() - 4)) return -3;
  size_t pos = 4;
  uint64_t cur, wrk, ep, cnt;
  uint8_t sh;
  memcpy(&cur, buf.data() + pos, 8); pos += 8;
  memcpy(&wrk, buf.data() + pos, 8); pos += 8;
  memcpy(&ep, buf.data() + pos, 8); pos += 8;
  sh = buf[pos]; pos += 1;
  memcpy(&cnt, buf.data() + pos, 8); pos += 8;
  if (pos + cnt * 8 + 4 != buf.size()) return -2;
  if (cnt != d->n) return -4;
  std::vector<uint64_t> idx(cnt);
  memcpy(idx.data(), buf.data() + pos, cnt * 8);
  for (uint64_t v : idx) if (v >= d->n) return -2;
  std::lock_guard<std::mutex> lk(d->mu);
  d->generation++;
  d->queue.clear();
  d->indices.swap(idx);
  d->current_index = cur;
  d->worker_index = cur;
  d->epoch_id = ep;
  d->shuffle = sh != 0;
  d->worker_done = false;
  d->cv.notify_all();
  (void)wrk;
  return 0;
}

}  // extern "C"
