// Rendezvous and liveness: a small TCP key-value store (rank 0 serves, every rank connects) and a file
// store with the same operations, plus heartbeats so that a rank that stopped answering is noticed on the
// host before the next collective is launched.
//
// The reference bootstraps through a rank-0 TCP star (src/distributed/distributed.cpp:49-183) and exchanges
// the NCCL id through a rendezvous file polled 3000 x 20 ms (:824-859); it has no heartbeat, no timeout on a
// collective and no rank-failure handling.  Here every blocking call takes a timeout and returns an error
// code instead of spinning forever, and `lt_store_dead_ranks` lists ranks whose heartbeat is older than a TTL.
//
// Wire protocol (one request per message, little-endian): u8 op, u32 key_len, key, u64 val_len, val.
//   op 1 SET -> u8 ok          op 2 GET -> u8 found, u64 len, bytes       op 3 ADD(i64 delta) -> i64 value
//   op 4 HEARTBEAT(rank in key) -> u8 ok     op 5 AGES -> u32 n, n x (i32 rank, i64 age_ms)
#include "lt_host.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

bool send_all(int fd, const void* p, size_t n) {
  const char* c = static_cast<const char*>(p);
  while (n) {
    ssize_t k = ::send(fd, c, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    c += k; n -= size_t(k);
  }
  return true;
}
bool recv_all(int fd, void* p, size_t n, int timeout_ms) {
  char* c = static_cast<char*>(p);
  const int64_t deadline = now_ms() + timeout_ms;
  while (n) {
    struct pollfd pfd{fd, POLLIN, 0};
    const int64_t left = deadline - now_ms();
    if (timeout_ms >= 0 && left <= 0) return false;
    const int pr = ::poll(&pfd, 1, timeout_ms < 0 ? -1 : int(left));
    if (pr <= 0) return false;
    ssize_t k = ::recv(fd, c, n, 0);
    if (k <= 0) return false;
    c += k; n -= size_t(k);
  }
  return true;
}

struct Server {
  int listen_fd = -1;
  int port = 0;
  std::atomic<bool> stop{false};
  std::thread accept_thread;
  std::vector<std::thread> workers;
  std::vector<int> client_fds;
  std::mutex mu;
  std::map<std::string, std::string> kv;
  std::map<int, int64_t> beats;

  void serve(int fd) {
    for (;;) {
      uint8_t op;
      if (!recv_all(fd, &op, 1, -1)) break;
      uint32_t klen;
      uint64_t vlen;
      if (!recv_all(fd, &klen, 4, 5000) || klen > (1u << 20)) break;
      std::string key(klen, '\0');
      if (klen && !recv_all(fd, &key[0], klen, 5000)) break;
      if (!recv_all(fd, &vlen, 8, 5000) || vlen > (1ull << 30)) break;
      std::string val(vlen, '\0');
      if (vlen && !recv_all(fd, &val[0], vlen, 30000)) break;
      if (op == 1) {
        { std::lock_guard<std::mutex> lk(mu); kv[key] = val; }
        uint8_t ok = 1;
        if (!send_all(fd, &ok, 1)) break;
      } else if (op == 2) {
        std::string out;
        uint8_t found = 0;
        { std::lock_guard<std::mutex> lk(mu); auto it = kv.find(key); if (it != kv.end()) { found = 1; out = it->second; } }
        uint64_t n = out.size();
        if (!send_all(fd, &found, 1) || !send_all(fd, &n, 8) || (n && !send_all(fd, out.data(), n))) break;
      } else if (op == 3) {
        int64_t delta = 0, cur = 0;
        if (val.size() == 8) memcpy(&delta, val.data(), 8);
        {
          std::lock_guard<std::mutex> lk(mu);
          auto it = kv.find(key);
          if (it != kv.end() && it->second.size() == 8) memcpy(&cur, it->second.data(), 8);
          cur += delta;
          kv[key] = std::string(reinterpret_cast<const char*>(&cur), 8);
        }
        if (!send_all(fd, &cur, 8)) break;
      } else if (op == 4) {
        { std::lock_guard<std::mutex> lk(mu); beats[std::atoi(key.c_str())] = now_ms(); }
        uint8_t ok = 1;
        if (!send_all(fd, &ok, 1)) break;
      } else if (op == 5) {
        std::vector<std::pair<int32_t, int64_t>> ages;
        { std::lock_guard<std::mutex> lk(mu); const int64_t t = now_ms(); for (auto& b : beats) ages.push_back({b.first, t - b.second}); }
        uint32_t n = uint32_t(ages.size());
        if (!send_all(fd, &n, 4)) break;
        bool ok = true;
        for (auto& a : ages) ok = ok && send_all(fd, &a.first, 4) && send_all(fd, &a.second, 8);
        if (!ok) break;
      } else {
        break;
      }
    }
    {
      // forget the descriptor before closing it: the number may be reused by another socket of the process at
      // once, and the stop path must not shut that one down
      std::lock_guard<std::mutex> lk(mu);
      for (auto it = client_fds.begin(); it != client_fds.end(); ++it)
        if (*it == fd) { client_fds.erase(it); break; }
    }
    ::close(fd);
  }
};

struct Client {
  int fd = -1;
  std::mutex mu;
  int timeout_ms = 30000;
  // After a failed send or a receive that timed out the stream is in the middle of a message: the next request would
  // read the tail of the old answer.  The connection is closed instead and every later call fails at once.
  void drop() {
    if (fd >= 0) ::close(fd);
    fd = -1;
  }
  bool request(uint8_t op, const std::string& key, const void* val, uint64_t vlen) {
    if (fd < 0) return false;
    uint32_t klen = uint32_t(key.size());
    const bool ok = send_all(fd, &op, 1) && send_all(fd, &klen, 4) && (klen == 0 || send_all(fd, key.data(), klen)) &&
                    send_all(fd, &vlen, 8) && (vlen == 0 || send_all(fd, val, vlen));
    if (!ok) drop();
    return ok;
  }
  bool recv(void* p, size_t n) {
    if (fd < 0) return false;
    const bool ok = recv_all(fd, p, n, timeout_ms);
    if (!ok) drop();
    return ok;
  }
};

}  // namespace

extern "C" {

// Starts the server on `port` (0 = pick one). Returns a handle, or nullptr; *port_out receives the bound port.
void* lt_store_server_start(int port, int* port_out) {
  int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return nullptr;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_ANY);
  addr.sin_port = htons(uint16_t(port));
  if (::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, 128) != 0) { ::close(fd); return nullptr; }
  socklen_t len = sizeof(addr);
  getsockname(fd, reinterpret_cast<sockaddr*>(&addr), &len);
  Server* s = new Server();
  s->listen_fd = fd;
  s->port = ntohs(addr.sin_port);
  if (port_out) *port_out = s->port;
  s->accept_thread = std::thread([s] {
    while (!s->stop) {
      struct pollfd pfd{s->listen_fd, POLLIN, 0};
      if (::poll(&pfd, 1, 100) <= 0) continue;
      int c = ::accept(s->listen_fd, nullptr, nullptr);
      if (c < 0) continue;
      int one2 = 1;
      setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one2, sizeof(one2));
      std::lock_guard<std::mutex> lk(s->mu);
      s->client_fds.push_back(c);
      s->workers.emplace_back([s, c] { s->serve(c); });
    }
  });
  return s;
}
void lt_store_server_stop(void* h) {
  Server* s = static_cast<Server*>(h);
  s->stop = true;
  if (s->accept_thread.joinable()) s->accept_thread.join();
  {
    std::lock_guard<std::mutex> lk(s->mu);
    for (int c : s->client_fds) ::shutdown(c, SHUT_RDWR);
  }
  for (auto& w : s->workers) if (w.joinable()) w.join();
  ::close(s->listen_fd);
  delete s;
}

// Connects with retries until timeout_ms has elapsed.
void* lt_store_connect(const char* host, int port, int timeout_ms) {
  const int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return nullptr;
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(uint16_t(port));
    if (inet_pton(AF_INET, host, &addr.sin_addr) != 1) { ::close(fd); return nullptr; }
    if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      Client* c = new Client();
      c->fd = fd;
      return c;
    }
    ::close(fd);
    if (now_ms() >= deadline) return nullptr;
    usleep(50 * 1000);
  }
}
void lt_store_close(void* h) {
  Client* c = static_cast<Client*>(h);
  if (c->fd >= 0) ::close(c->fd);
  delete c;
}

int lt_store_set(void* h, const char* key, const void* val, uint64_t len) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  uint8_t ok = 0;
  if (!c->request(1, key, val, len) || !c->recv(&ok, 1)) return -1;
  return ok ? 0 : -2;
}
// Polls until the key exists or timeout_ms passed. Returns the value length (copied up to cap), -1 on I/O
// error, -2 on timeout.
int64_t lt_store_get(void* h, const char* key, void* buf, uint64_t cap, int timeout_ms) {
  Client* c = static_cast<Client*>(h);
  const int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    {
      std::lock_guard<std::mutex> lk(c->mu);
      uint8_t found;
      uint64_t n;
      if (!c->request(2, key, nullptr, 0) || !c->recv(&found, 1) || !c->recv(&n, 8)) return -1;
      std::string tmp(n, '\0');
      if (n && !c->recv(&tmp[0], n)) return -1;
      if (found) {
        memcpy(buf, tmp.data(), n < cap ? n : cap);
        return int64_t(n);
      }
    }
    if (now_ms() >= deadline) return -2;
    usleep(5 * 1000);
  }
}
int64_t lt_store_add(void* h, const char* key, int64_t delta) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  int64_t out = 0;
  if (!c->request(3, key, &delta, 8) || !c->recv(&out, 8)) return INT64_MIN;
  return out;
}
int lt_store_heartbeat(void* h, int rank) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  uint8_t ok = 0;
  const std::string key = std::to_string(rank);
  if (!c->request(4, key, nullptr, 0) || !c->recv(&ok, 1)) return -1;
  return 0;
}
// Time a client waits for the answer to one request (default 30 s).
void lt_store_set_timeout(void* h, int timeout_ms) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  c->timeout_ms = timeout_ms;
}
// 1 while the connection is usable, 0 after an I/O error or a timeout closed it.
int lt_store_alive(void* h) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  return c->fd >= 0 ? 1 : 0;
}
// Ranks of [0, world) with no heartbeat at all, or whose last beat is older than ttl_ms.  A rank that died before its
// first beat is only visible this way; the caller applies its own grace period after start-up.  Returns the count.
int lt_store_silent_ranks(void* h, int world, int ttl_ms, int32_t* ranks, int cap) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  uint32_t n;
  if (!c->request(5, "", nullptr, 0) || !c->recv(&n, 4)) return -1;
  std::vector<int64_t> age(size_t(world > 0 ? world : 0), -1);
  for (uint32_t i = 0; i < n; ++i) {
    int32_t r;
    int64_t a;
    if (!c->recv(&r, 4) || !c->recv(&a, 8)) return -1;
    if (r >= 0 && r < world) age[size_t(r)] = a;
  }
  int out = 0;
  for (int r = 0; r < world; ++r)
    if ((age[size_t(r)] < 0 || age[size_t(r)] > ttl_ms) && out < cap) ranks[out++] = r;
  return out;
}
// Ranks (among those that ever sent a heartbeat) whose last beat is older than ttl_ms. Returns the count.
int lt_store_dead_ranks(void* h, int ttl_ms, int32_t* ranks, int cap) {
  Client* c = static_cast<Client*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  uint32_t n;
  if (!c->request(5, "", nullptr, 0) || !c->recv(&n, 4)) return -1;
  int out = 0;
  for (uint32_t i = 0; i < n; ++i) {
    int32_t r;
    int64_t age;
    if (!c->recv(&r, 4) || !c->recv(&age, 8)) return -1;
    if (age > ttl_ms && out < cap) ranks[out++] = r;
  }
  return out;
}
// Barrier over the store: every rank adds 1 to `key` and waits until it reaches world * generation.
int lt_store_barrier(void* h, const char* key, int world, int timeout_ms) {
  const int64_t mine = lt_store_add(h, key, 1);
  if (mine == INT64_MIN) return -1;
  const int64_t target = (mine + world - 1) / world * world;
  const int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    const int64_t cur = lt_store_add(h, key, 0);
    if (cur == INT64_MIN) return -1;
    if (cur >= target) return 0;
    if (now_ms() >= deadline) {
      // take this rank's arrival back: otherwise the counter stays off a multiple of `world` and every later
      // barrier on the key releases early or never
      lt_store_add(h, key, -1);
      return -2;
    }
    usleep(2 * 1000);
  }
}

// ------------------------------------------------------------------ file store (shared directory)
int lt_filestore_set(const char* dir, const char* key, const void* val, uint64_t len) {
  ::mkdir(dir, 0777);
  const std::string final_path = std::string(dir) + "/" + key;
  const std::string tmp = final_path + ".tmp." + std::to_string(::getpid());
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return -1;
  const bool ok = fwrite(val, 1, len, f) == len;
  fclose(f);
  if (!ok) { ::unlink(tmp.c_str()); return -1; }
  return ::rename(tmp.c_str(), final_path.c_str()) == 0 ? 0 : -1;
}
int64_t lt_filestore_get(const char* dir, const char* key, void* buf, uint64_t cap, int timeout_ms) {
  const std::string path = std::string(dir) + "/" + key;
  const int64_t deadline = now_ms() + timeout_ms;
  for (;;) {
    FILE* f = fopen(path.c_str(), "rb");
    if (f) {
      fseek(f, 0, SEEK_END);
      long sz = ftell(f);
      fseek(f, 0, SEEK_SET);
      std::vector<char> tmp(sz > 0 ? size_t(sz) : 0);
      const size_t got = sz > 0 ? fread(tmp.data(), 1, size_t(sz), f) : 0;
      fclose(f);
      memcpy(buf, tmp.data(), got < cap ? got : cap);
      return int64_t(got);
    }
    if (now_ms() >= deadline) return -2;
    usleep(20 * 1000);
  }
}

}  // extern "C"
