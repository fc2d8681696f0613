// Token-stream loader for language-model training: a flat binary file of token ids (uint16 or uint32, little endian)
// is memory-mapped and cut into windows of seq_len + 1 consecutive tokens (window i starts at token i * seq_len, so the
// target of a window's last input is the first input of the next window).  Every epoch the windows are permuted with a
// generator seeded by (seed, epoch); rank r of `world` takes positions r, r + world, ... of the permutation, so the ranks
// see disjoint windows and every rank gets the same number of batches (the remainder is dropped).  A worker thread
// widens the tokens to int64 straight into queue buffers; `lt_ts_next` copies one batch into the caller's (pinned)
// tensors.  The position is (epoch, batch index) and nothing else, so a resumed job continues with exactly the batches
// the interrupted one would have seen: `lt_ts_seek`.
//
// The reference has no counterpart (its loader serves rows of two in-memory float tensors, src/data/data.cpp).
#include "lt_host.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <deque>
#include <mutex>
#include <random>
#include <thread>
#include <vector>

namespace {

struct TsBatch {
  std::vector<int64_t> tok, tgt;
  uint64_t generation = 0;
  bool end_of_epoch = false;
};

struct TokenStream {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  int token_bytes = 2;
  uint64_t n_tokens = 0, seq_len = 0, batch = 0, n_windows = 0, batches_per_epoch = 0;
  bool shuffle = false;
  uint64_t seed = 0;
  int rank = 0, world = 1;
  size_t prefetch = 2;

  std::vector<uint64_t> perm;      // this epoch's order of all windows
  uint64_t epoch = 0;
  uint64_t consumer_pos = 0;       // batches handed out in this epoch
  uint64_t worker_pos = 0;         // batches assembled in this epoch
  uint64_t generation = 0;         // bumped by reset / seek: batches of an older generation are dropped
  bool worker_done = false;
  bool stop = false;
  std::deque<TsBatch> queue;
  std::mutex mu;
  std::condition_variable cv;
  std::thread worker;

  void make_perm() {
    perm.resize(n_windows);
    for (uint64_t i = 0; i < n_windows; ++i) perm[i] = i;
    if (shuffle) {
      std::mt19937_64 rng(seed + epoch * 0x9E3779B97F4A7C15ull);
      std::shuffle(perm.begin(), perm.end(), rng);
    }
  }

  inline int64_t token_at(uint64_t i) const {
    if (token_bytes == 2) { uint16_t v; memcpy(&v, map + i * 2, 2); return v; }
    uint32_t v; memcpy(&v, map + i * 4, 4); return v;
  }

  void fill(TsBatch& b, uint64_t batch_index, const std::vector<uint64_t>& order) const {
    b.tok.resize(batch * seq_len);
    b.tgt.resize(batch * seq_len);
    for (uint64_t r = 0; r < batch; ++r) {
      const uint64_t slot = (batch_index * batch + r) * uint64_t(world) + uint64_t(rank);
      const uint64_t start = order[slot] * seq_len;
      int64_t* t = b.tok.data() + r * seq_len;
      int64_t* g = b.tgt.data() + r * seq_len;
      int64_t cur = token_at(start);
      for (uint64_t j = 0; j < seq_len; ++j) {
        const int64_t nxt = token_at(start + j + 1);
        t[j] = cur;
        g[j] = nxt;
        cur = nxt;
      }
    }
  }

  void run() {
    std::unique_lock<std::mutex> lk(mu);
    while (!stop) {
      cv.wait(lk, [&] { return stop || (!worker_done && queue.size() < prefetch); });
      if (stop) break;
      const uint64_t gen = generation;
      const uint64_t index = worker_pos;
      TsBatch b;
      b.generation = gen;
      if (index >= batches_per_epoch) {
        worker_done = true;
        b.end_of_epoch = true;
        queue.push_back(std::move(b));
        cv.notify_all();
        continue;
      }
      const std::vector<uint64_t> order = perm;   // the copy is cheap next to the batch and lets reset run meanwhile
      lk.unlock();
      fill(b, index, order);
      lk.lock();
      if (gen != generation) continue;            // reset or seek happened while this batch was assembled
      worker_pos = index + 1;
      queue.push_back(std::move(b));
      cv.notify_all();
    }
  }

  void restart_locked(uint64_t new_epoch, uint64_t position) {
    epoch = new_epoch;
    make_perm();
    consumer_pos = worker_pos = std::min(position, batches_per_epoch);
    worker_done = false;
    ++generation;
    queue.clear();
    cv.notify_all();
  }
};

}  // namespace

extern "C" {

// token_bytes: 2 or 4.  Returns nullptr when the file cannot be mapped, holds fewer than seq_len + 1 tokens, or the
// arguments make no batch (batch * world windows are needed for one).
void* lt_ts_open(const char* path, int token_bytes, uint64_t seq_len, uint64_t batch, int shuffle, uint64_t seed, int rank,
                 int world, int prefetch) {
  if ((token_bytes != 2 && token_bytes != 4) || seq_len == 0 || batch == 0 || world < 1 || rank < 0 || rank >= world) return nullptr;
  const int fd = ::open(path, O_RDONLY);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < off_t((seq_len + 1) * uint64_t(token_bytes))) { ::close(fd); return nullptr; }
  void* m = mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { ::close(fd); return nullptr; }
  TokenStream* s = new TokenStream();
  s->fd = fd;
  s->map = static_cast<const uint8_t*>(m);
  s->map_bytes = size_t(st.st_size);
  s->token_bytes = token_bytes;
  s->n_tokens = uint64_t(st.st_size) / uint64_t(token_bytes);
  s->seq_len = seq_len;
  s->batch = batch;
  s->n_windows = (s->n_tokens - 1) / seq_len;
  s->batches_per_epoch = (s->n_windows / uint64_t(world)) / batch;
  s->shuffle = shuffle != 0;
  s->seed = seed;
  s->rank = rank;
  s->world = world;
  s->prefetch = size_t(prefetch < 1 ? 1 : prefetch);
  if (s->batches_per_epoch == 0) {
    munmap(m, s->map_bytes);
    ::close(fd);
    delete s;
    return nullptr;
  }
  s->make_perm();
  s->worker = std::thread([s] { s->run(); });
  return s;
}

void lt_ts_close(void* h) {
  if (!h) return;
  TokenStream* s = static_cast<TokenStream*>(h);
  {
    std::lock_guard<std::mutex> lk(s->mu);
    s->stop = true;
  }
  s->cv.notify_all();
  if (s->worker.joinable()) s->worker.join();
  munmap(const_cast<uint8_t*>(s->map), s->map_bytes);
  ::close(s->fd);
  delete s;
}

uint64_t lt_ts_num_tokens(void* h) { return static_cast<TokenStream*>(h)->n_tokens; }
uint64_t lt_ts_num_windows(void* h) { return static_cast<TokenStream*>(h)->n_windows; }
uint64_t lt_ts_batches_per_epoch(void* h) { return static_cast<TokenStream*>(h)->batches_per_epoch; }

uint64_t lt_ts_epoch(void* h) {
  TokenStream* s = static_cast<TokenStream*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  return s->epoch;
}

uint64_t lt_ts_position(void* h) {
  TokenStream* s = static_cast<TokenStream*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  return s->consumer_pos;
}

// Copies the next batch ([batch, seq_len] int64 each) and returns 1; returns 0 at the end of the epoch (call
// lt_ts_next_epoch to go on).
int lt_ts_next(void* h, int64_t* tokens_out, int64_t* targets_out) {
  TokenStream* s = static_cast<TokenStream*>(h);
  std::unique_lock<std::mutex> lk(s->mu);
  for (;;) {
    s->cv.wait(lk, [&] { return s->stop || !s->queue.empty(); });
    if (s->stop) return 0;
    TsBatch b = std::move(s->queue.front());
    s->queue.pop_front();
    s->cv.notify_all();
    if (b.generation != s->generation) continue;
    if (b.end_of_epoch) {
      // leave the marker's meaning in place for repeated calls: the worker stays done until the next epoch starts
      TsBatch again;
      again.generation = s->generation;
      again.end_of_epoch = true;
      s->queue.push_front(std::move(again));
      return 0;
    }
    s->consumer_pos += 1;
    lk.unlock();
    const size_t bytes = size_t(s->batch * s->seq_len) * sizeof(int64_t);
    memcpy(tokens_out, b.tok.data(), bytes);
    memcpy(targets_out, b.tgt.data(), bytes);
    return 1;
  }
}

// Starts the next epoch (a new permutation when shuffling).
void lt_ts_next_epoch(void* h) {
  TokenStream* s = static_cast<TokenStream*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->restart_locked(s->epoch + 1, 0);
}

// Jumps to batch `position` of epoch `epoch` (what lt_ts_epoch / lt_ts_position returned when a checkpoint was taken).
void lt_ts_seek(void* h, uint64_t epoch, uint64_t position) {
  TokenStream* s = static_cast<TokenStream*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->restart_locked(epoch, position);
}

}  // extern "C"
