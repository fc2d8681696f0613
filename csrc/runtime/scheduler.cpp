// Serving runtime on the host: continuous-batching scheduler with a paged KV block manager, a token-prefix
// cache keyed by a rolling hash, and the guided-decoding vocabulary mask.
//
// The scheduling policy follows the reference (src/llm/continuous_batching.cpp:9-197): FIFO admission while
// enough free KV blocks exist for prompt + max_new_tokens (reserved up front), a per-step token budget,
// chunked prefill, one token per running sequence in the batched decode, greedy sampling done by the
// caller, stop on EOS or max_new_tokens, blocks recycled on completion.  The model stays outside: `plan`
// returns what to run this step, `commit_*` feeds the sampled tokens back.
// Guided decoding follows src/llm/guided_decoding.cpp:8-65 ("digits", "prefix:<s>", "regex:<re>").
#include "lt_host.h"

#include <algorithm>
#include <cctype>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <regex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Req {
  int64_t id;
  std::vector<int32_t> prompt;
  std::vector<int32_t> generated;
  int max_new;
  int prefill_done = 0;
  int planned_chunk = 0;
  bool finished = false;
  std::vector<int32_t> blocks;
};

struct Sched {
  int num_blocks, block_size, max_seqs, max_tokens, eos_id;
  std::vector<int32_t> free_blocks;
  std::deque<std::shared_ptr<Req>> pending;
  std::vector<std::shared_ptr<Req>> running;
  std::vector<std::shared_ptr<Req>> done;
  std::unordered_map<int64_t, std::shared_ptr<Req>> by_id;
  std::mutex mu;

  void finish(const std::shared_ptr<Req>& r) {
    r->finished = true;
    for (int32_t b : r->blocks) free_blocks.push_back(b);
    r->blocks.clear();
    running.erase(std::remove(running.begin(), running.end(), r), running.end());
    done.push_back(r);
  }
};

struct PrefixEntry {
  std::vector<int32_t> tokens;
  std::vector<int32_t> blocks;
  uint64_t last_use;
};
struct PrefixCache {
  std::unordered_map<uint64_t, PrefixEntry> map;
  uint64_t clock = 0;
  size_t capacity;
  std::mutex mu;
};

uint64_t hash_tokens(const int32_t* t, int n) {
  uint64_t h = 1469598103934665603ull;
  for (int i = 0; i < n; ++i) {
    h ^= uint64_t(uint32_t(t[i]));
    h *= 1099511628211ull;
  }
  return h;
}

}  // namespace

extern "C" {

void* lt_sched_create(int num_blocks, int block_size, int max_num_seqs, int max_num_batched_tokens, int eos_id) {
  Sched* s = new Sched();
  s->num_blocks = num_blocks; s->block_size = block_size; s->max_seqs = max_num_seqs;
  s->max_tokens = max_num_batched_tokens; s->eos_id = eos_id;
  for (int i = num_blocks - 1; i >= 0; --i) s->free_blocks.push_back(i);
  return s;
}
void lt_sched_destroy(void* h) { delete static_cast<Sched*>(h); }

int lt_sched_add_request(void* h, int64_t id, const int32_t* prompt, int prompt_len, int max_new_tokens) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  if (s->by_id.count(id)) return -1;
  auto r = std::make_shared<Req>();
  r->id = id;
  r->prompt.assign(prompt, prompt + prompt_len);
  r->max_new = max_new_tokens;
  s->by_id[id] = r;
  s->pending.push_back(r);
  return 0;
}

// Admits pending requests, then plans one step.  For every active request i: req_ids[i], chunk_start[i],
// chunk_len[i] (> 0: prefill that slice of the prompt; 0: decode one token).  Returns the number of entries.
int lt_sched_plan(void* h, int64_t* req_ids, int32_t* chunk_start, int32_t* chunk_len, int cap) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  while (int(s->running.size()) < s->max_seqs && !s->pending.empty()) {
    auto r = s->pending.front();
    const size_t total = r->prompt.size() + size_t(r->max_new);
    const size_t need = (total + s->block_size - 1) / s->block_size;
    if (s->free_blocks.size() < need) break;
    s->pending.pop_front();
    for (size_t i = 0; i < need; ++i) {
      r->blocks.push_back(s->free_blocks.back());
      s->free_blocks.pop_back();
    }
    s->running.push_back(r);
  }
  int budget = s->max_tokens;
  int n = 0;
  for (auto& r : s->running) {
    if (budget <= 0 || n >= cap) break;
    req_ids[n] = r->id;
    const int left = int(r->prompt.size()) - r->prefill_done;
    if (left > 0) {
      const int chunk = std::min(left, budget);
      chunk_start[n] = r->prefill_done;
      chunk_len[n] = chunk;
      r->planned_chunk = chunk;
      budget -= chunk;
    } else {
      chunk_start[n] = int(r->prompt.size() + r->generated.size()) - 1;
      chunk_len[n] = 0;
      r->planned_chunk = 0;
      budget -= 1;
    }
    ++n;
  }
  return n;
}

// After a prefill chunk ran: token = argmax of the last position when the chunk completed the prompt, else -1.
int lt_sched_commit(void* h, int64_t id, int32_t token) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->by_id.find(id);
  if (it == s->by_id.end()) return -1;
  auto r = it->second;
  if (r->finished) return -2;
  if (r->planned_chunk > 0) {
    r->prefill_done += r->planned_chunk;
    r->planned_chunk = 0;
    if (r->prefill_done < int(r->prompt.size())) return 0;  // more prompt to go; no token yet
  }
  if (token >= 0) {
    r->generated.push_back(token);
    if (token == s->eos_id || int(r->generated.size()) >= r->max_new) s->finish(r);
  }
  return 0;
}

int lt_sched_tokens(void* h, int64_t id, int32_t* out, int cap, int* prompt_len) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->by_id.find(id);
  if (it == s->by_id.end()) return -1;
  auto r = it->second;
  int n = 0;
  for (int32_t t : r->prompt) if (n < cap) out[n++] = t;
  for (int32_t t : r->generated) if (n < cap) out[n++] = t;
  if (prompt_len) *prompt_len = int(r->prompt.size());
  return int(r->prompt.size() + r->generated.size());
}

int lt_sched_block_table(void* h, int64_t id, int32_t* out, int cap) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->by_id.find(id);
  if (it == s->by_id.end()) return -1;
  int n = 0;
  for (int32_t b : it->second->blocks) if (n < cap) out[n++] = b;
  return int(it->second->blocks.size());
}

int lt_sched_context_len(void* h, int64_t id) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  auto it = s->by_id.find(id);
  if (it == s->by_id.end()) return -1;
  return it->second->prefill_done + int(it->second->generated.size());
}

// Pops finished requests; returns how many ids were written.
int lt_sched_pop_finished(void* h, int64_t* ids, int cap) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  int n = 0;
  while (!s->done.empty() && n < cap) {
    ids[n++] = s->done.front()->id;
    s->done.erase(s->done.begin());
  }
  return n;
}
void lt_sched_release(void* h, int64_t id) {
  Sched* s = static_cast<Sched*>(h);
  std::lock_guard<std::mutex> lk(s->mu);
  s->by_id.erase(id);
}
int lt_sched_num_free_blocks(void* h) { Sched* s = static_cast<Sched*>(h); std::lock_guard<std::mutex> lk(s->mu); return int(s->free_blocks.size()); }
int lt_sched_num_running(void* h) { Sched* s = static_cast<Sched*>(h); std::lock_guard<std::mutex> lk(s->mu); return int(s->running.size()); }
int lt_sched_num_pending(void* h) { Sched* s = static_cast<Sched*>(h); std::lock_guard<std::mutex> lk(s->mu); return int(s->pending.size()); }

// ------------------------------------------------------------------ prefix cache (token prefix -> KV blocks)
void* lt_prefix_create(int capacity) {
  PrefixCache* c = new PrefixCache();
  c->capacity = capacity > 0 ? size_t(capacity) : 1024;
  return c;
}
void lt_prefix_destroy(void* h) { delete static_cast<PrefixCache*>(h); }
int lt_prefix_insert(void* h, const int32_t* tokens, int n, const int32_t* blocks, int n_blocks) {
  PrefixCache* c = static_cast<PrefixCache*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->map.size() >= c->capacity) {  // evict the least recently used entry
    auto victim = c->map.begin();
    for (auto it = c->map.begin(); it != c->map.end(); ++it)
      if (it->second.last_use < victim->second.last_use) victim = it;
    c->map.erase(victim);
  }
  PrefixEntry e;
  e.tokens.assign(tokens, tokens + n);
  e.blocks.assign(blocks, blocks + n_blocks);
  e.last_use = ++c->clock;
  c->map[hash_tokens(tokens, n)] = std::move(e);
  return 0;
}
// Longest cached prefix of `tokens` whose length is a multiple of `granularity`; writes its blocks.
int lt_prefix_lookup(void* h, const int32_t* tokens, int n, int granularity, int32_t* blocks, int cap, int* n_blocks) {
  PrefixCache* c = static_cast<PrefixCache*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  if (granularity <= 0) granularity = 1;
  for (int len = n / granularity * granularity; len > 0; len -= granularity) {
    auto it = c->map.find(hash_tokens(tokens, len));
    if (it == c->map.end()) continue;
    if (int(it->second.tokens.size()) != len || memcmp(it->second.tokens.data(), tokens, len * sizeof(int32_t)) != 0) continue;
    it->second.last_use = ++c->clock;
    int k = 0;
    for (int32_t b : it->second.blocks) if (k < cap) blocks[k++] = b;
    *n_blocks = int(it->second.blocks.size());
    return len;
  }
  *n_blocks = 0;
  return 0;
}
int lt_prefix_size(void* h) { PrefixCache* c = static_cast<PrefixCache*>(h); std::lock_guard<std::mutex> lk(c->mu); return int(c->map.size()); }

// ------------------------------------------------------------------ guided decoding
// allowed[v] = 1 when vocabulary entry v may follow `prefix` under `pattern`.
// vocab_blob: the vocabulary strings concatenated; vocab_off[v]..vocab_off[v+1] delimit entry v.
int lt_guided_mask(const char* pattern_c, const char* prefix_c, const char* vocab_blob, const int64_t* vocab_off, int V,
                   uint8_t* allowed) {
  const std::string target(pattern_c), prefix(prefix_c);
  const bool is_regex = target.rfind("regex:", 0) == 0;
  const std::string pattern = is_regex ? target.substr(6) : target;
  std::regex re;
  bool regex_ok = true;
  if (is_regex) {
    try { re = std::regex(pattern); } catch (...) { regex_ok = false; }
  }
  const bool is_prefix = !is_regex && pattern.rfind("prefix:", 0) == 0;
  const std::string want = is_prefix ? pattern.substr(7) : std::string();
  for (int v = 0; v < V; ++v) {
    const std::string cand = prefix + std::string(vocab_blob + vocab_off[v], size_t(vocab_off[v + 1] - vocab_off[v]));
    bool ok = true;
    if (is_regex) {
      ok = regex_ok && (std::regex_match(cand, re) || std::regex_search(cand, re));
    } else if (pattern == "digits") {
      for (char ch : cand) if (!std::isdigit(static_cast<unsigned char>(ch))) { ok = false; break; }
    } else if (is_prefix) {
      ok = (want.rfind(cand, 0) == 0) || (cand.rfind(want, 0) == 0);
    }
    allowed[v] = ok ? 1 : 0;
  }
  return 0;
}

}  // extern "C"
