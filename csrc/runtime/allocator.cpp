// Caching allocator core and LRU residency manager (host side, device-agnostic).
//
// The policy mirrors the reference: size-ordered free lists, a cached block is reused when it is at most
// twice the request, caches are capped and `empty_cache` returns everything to the system
// (src/memory_manager/allocator.cpp:43-142); storages register with an LRU manager that, when a new
// registration would exceed the limit, asks the least-recently-used idle storages to leave the device
// (src/memory_manager/memory_manager.cpp:54-107).  The raw allocate / release functions are supplied by the
// caller: malloc/free for host pools, and cudaMalloc/cudaFree (stream-ordered reuse handled by the CUDA-side
// wrapper) for device pools.  Unlike the reference (512 MB default), a pool has no default cap: 180 GB of
// HBM3e per GPU is there to be used, and a cap is opt-in.
#include "lt_host.h"

#include <cstdint>
#include <cstdlib>
#include <list>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

typedef void* (*RawAlloc)(uint64_t bytes, void* ctx);
typedef void (*RawFree)(void* ptr, void* ctx);

struct Pool {
  RawAlloc ralloc;
  RawFree rfree;
  void* ctx;
  uint64_t max_cached;      // bytes kept in the free lists (0 = unlimited)
  uint64_t max_block;       // blocks at least this large are never cached (0 = cache everything)
  uint64_t round_to;        // request sizes are rounded up to a multiple of this
  std::multimap<uint64_t, void*> free_blocks;
  std::unordered_map<void*, uint64_t> live;  // ptr -> rounded size
  uint64_t cached_bytes = 0, live_bytes = 0, peak_live = 0, n_alloc = 0, n_hit = 0, n_raw = 0;
  std::mutex mu;
};

void* host_alloc(uint64_t bytes, void*) { return std::malloc(bytes); }
void host_free(void* p, void*) { std::free(p); }

typedef int (*EvictFn)(uint64_t storage_id, void* ctx);

struct Lru {
  uint64_t limit;
  uint64_t used = 0;
  EvictFn evict;
  void* ctx;
  std::list<uint64_t> order;  // front = least recently used
  struct Entry { uint64_t bytes; bool in_use; std::list<uint64_t>::iterator it; };
  std::unordered_map<uint64_t, Entry> entries;
  uint64_t n_evictions = 0;
  std::mutex mu;
};

}  // namespace

extern "C" {

// ralloc/rfree == nullptr selects malloc/free.
void* lt_pool_create(void* ralloc, void* rfree, void* ctx, uint64_t max_cached, uint64_t max_block, uint64_t round_to) {
  Pool* p = new Pool();
  p->ralloc = ralloc ? reinterpret_cast<RawAlloc>(ralloc) : host_alloc;
  p->rfree = rfree ? reinterpret_cast<RawFree>(rfree) : host_free;
  p->ctx = ctx;
  p->max_cached = max_cached;
  p->max_block = max_block;
  p->round_to = round_to ? round_to : 512;
  return p;
}

void* lt_pool_alloc(void* h, uint64_t bytes) {
  Pool* p = static_cast<Pool*>(h);
  if (bytes == 0) bytes = 1;
  const uint64_t sz = (bytes + p->round_to - 1) / p->round_to * p->round_to;
  std::lock_guard<std::mutex> lk(p->mu);
  p->n_alloc++;
  auto it = p->free_blocks.lower_bound(sz);
  void* ptr = nullptr;
  uint64_t got = sz;
  if (it != p->free_blocks.end() && it->first <= 2 * sz) {  // best fit, at most twice the request
    ptr = it->second;
    got = it->first;
    p->cached_bytes -= got;
    p->free_blocks.erase(it);
    p->n_hit++;
  } else {
    ptr = p->ralloc(sz, p->ctx);
    p->n_raw++;
    if (!ptr) {
      // release the cache and retry once
      for (auto& b : p->free_blocks) p->rfree(b.second, p->ctx);
      p->free_blocks.clear();
      p->cached_bytes = 0;
      ptr = p->ralloc(sz, p->ctx);
      if (!ptr) return nullptr;
    }
  }
  p->live[ptr] = got;
  p->live_bytes += got;
  if (p->live_bytes > p->peak_live) p->peak_live = p->live_bytes;
  return ptr;
}

int lt_pool_free(void* h, void* ptr) {
  Pool* p = static_cast<Pool*>(h);
  if (!ptr) return 0;
  std::lock_guard<std::mutex> lk(p->mu);
  auto it = p->live.find(ptr);
  if (it == p->live.end()) return -1;
  const uint64_t sz = it->second;
  p->live.erase(it);
  p->live_bytes -= sz;
  const bool too_big = p->max_block && sz >= p->max_block;
  const bool over_cap = p->max_cached && p->cached_bytes + sz > p->max_cached;
  if (too_big || over_cap) {
    p->rfree(ptr, p->ctx);
  } else {
    p->free_blocks.emplace(sz, ptr);
    p->cached_bytes += sz;
  }
  return 0;
}

void lt_pool_empty_cache(void* h) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  for (auto& b : p->free_blocks) p->rfree(b.second, p->ctx);
  p->free_blocks.clear();
  p->cached_bytes = 0;
}
void lt_pool_set_max_cached(void* h, uint64_t bytes) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  p->max_cached = bytes;
  while (p->max_cached && p->cached_bytes > p->max_cached && !p->free_blocks.empty()) {
    auto it = std::prev(p->free_blocks.end());
    p->rfree(it->second, p->ctx);
    p->cached_bytes -= it->first;
    p->free_blocks.erase(it);
  }
}
// stats: {cached_bytes, live_bytes, peak_live, n_alloc, n_cache_hits, n_raw_allocs}
void lt_pool_stats(void* h, uint64_t* out6) {
  Pool* p = static_cast<Pool*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  out6[0] = p->cached_bytes; out6[1] = p->live_bytes; out6[2] = p->peak_live;
  out6[3] = p->n_alloc; out6[4] = p->n_hit; out6[5] = p->n_raw;
}
void lt_pool_destroy(void* h) {
  Pool* p = static_cast<Pool*>(h);
  lt_pool_empty_cache(h);
  delete p;
}

// ------------------------------------------------------------------ LRU residency manager
void* lt_lru_create(uint64_t limit_bytes, void* evict_fn, void* ctx) {
  Lru* l = new Lru();
  l->limit = limit_bytes;
  l->evict = reinterpret_cast<EvictFn>(evict_fn);
  l->ctx = ctx;
  return l;
}
void lt_lru_destroy(void* h) { delete static_cast<Lru*>(h); }
void lt_lru_set_limit(void* h, uint64_t bytes) { Lru* l = static_cast<Lru*>(h); std::lock_guard<std::mutex> lk(l->mu); l->limit = bytes; }
uint64_t lt_lru_used(void* h) { Lru* l = static_cast<Lru*>(h); std::lock_guard<std::mutex> lk(l->mu); return l->used; }
uint64_t lt_lru_evictions(void* h) { Lru* l = static_cast<Lru*>(h); std::lock_guard<std::mutex> lk(l->mu); return l->n_evictions; }

// Registers a storage as resident; idle least-recently-used storages are evicted (callback) until it fits.
// Returns the number of storages evicted. Ids evicted are written to evicted[] (up to cap).
int lt_lru_register(void* h, uint64_t id, uint64_t bytes, uint64_t* evicted, int cap) {
  Lru* l = static_cast<Lru*>(h);
  std::vector<uint64_t> victims;
  {
    std::lock_guard<std::mutex> lk(l->mu);
    if (l->entries.count(id)) return 0;
    auto it = l->order.begin();
    while (l->limit && l->used + bytes > l->limit && it != l->order.end()) {
      auto e = l->entries.find(*it);
      if (e != l->entries.end() && !e->second.in_use) {
        victims.push_back(*it);
        l->used -= e->second.bytes;
        it = l->order.erase(it);
        l->entries.erase(e);
        l->n_evictions++;
      } else {
        ++it;
      }
    }
    l->order.push_back(id);
    l->entries[id] = Lru::Entry{bytes, false, std::prev(l->order.end())};
    l->used += bytes;
  }
  int n = 0;
  for (uint64_t v : victims) {
    if (l->evict) l->evict(v, l->ctx);
    if (n < cap) evicted[n] = v;
    ++n;
  }
  return n;
}
void lt_lru_unregister(void* h, uint64_t id) {
  Lru* l = static_cast<Lru*>(h);
  std::lock_guard<std::mutex> lk(l->mu);
  auto e = l->entries.find(id);
  if (e == l->entries.end()) return;
  l->used -= e->second.bytes;
  l->order.erase(e->second.it);
  l->entries.erase(e);
}
void lt_lru_touch(void* h, uint64_t id) {
  Lru* l = static_cast<Lru*>(h);
  std::lock_guard<std::mutex> lk(l->mu);
  auto e = l->entries.find(id);
  if (e == l->entries.end()) return;
  l->order.erase(e->second.it);
  l->order.push_back(id);
  e->second.it = std::prev(l->order.end());
}
void lt_lru_pin(void* h, uint64_t id, int in_use) {
  Lru* l = static_cast<Lru*>(h);
  std::lock_guard<std::mutex> lk(l->mu);
  auto e = l->entries.find(id);
  if (e != l->entries.end()) e->second.in_use = in_use != 0;
}

}  // extern "C"
