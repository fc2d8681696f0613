// NCCL without a framework in between: the library is opened at run time (the copy the process already holds, if any),
// the communicator id travels through the caller's rendezvous store, and collectives are enqueued on the caller's
// CUDA stream.  Counterpart of the reference's NCCLBridge (src/distributed/distributed.cpp:785-905: nine entry points
// resolved with dlsym, id exchanged through a file or TCP) - with the 128-byte id passed to ncclCommInitRank by value,
// which is what the library's ABI asks for.
#include "kernels/lt_cuda.h"
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace {

struct NcclId { char bytes[128]; };   // ncclUniqueId
typedef void* Comm;                   // ncclComm_t

struct Api {
  void* lib = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(Comm*, int, NcclId, int) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*GetVersion)(int*) = nullptr;
  bool ok = false;
};
Api g_api;
std::mutex g_mu;

template <class F>
bool sym(F& f, const char* name) {
  f = reinterpret_cast<F>(dlsym(g_api.lib, name));
  return f != nullptr;
}

bool load() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_api.ok) return true;
  // the copy that is already in the process (PyTorch links one) wins; otherwise the system's
  g_api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (!g_api.lib) g_api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!g_api.lib) g_api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!g_api.lib) return false;
  g_api.ok = sym(g_api.GetUniqueId, "ncclGetUniqueId") && sym(g_api.CommInitRank, "ncclCommInitRank") &&
             sym(g_api.CommDestroy, "ncclCommDestroy") && sym(g_api.AllReduce, "ncclAllReduce") &&
             sym(g_api.AllGather, "ncclAllGather") && sym(g_api.ReduceScatter, "ncclReduceScatter") &&
             sym(g_api.Broadcast, "ncclBroadcast") && sym(g_api.Send, "ncclSend") && sym(g_api.Recv, "ncclRecv") &&
             sym(g_api.GroupStart, "ncclGroupStart") && sym(g_api.GroupEnd, "ncclGroupEnd") && sym(g_api.GetVersion, "ncclGetVersion");
  return g_api.ok;
}

}  // namespace

extern "C" {

// 0 when the library cannot be opened, else its version code (e.g. 22809).
int lt_nccl_version() {
  if (!load()) return 0;
  int v = 0;
  g_api.GetVersion(&v);
  return v;
}
// Rank 0 creates the id (128 bytes) and publishes it through the rendezvous store.
int lt_nccl_unique_id(void* out128) {
  if (!load()) return -1;
  NcclId id;
  const int r = g_api.GetUniqueId(&id);
  if (r == 0) memcpy(out128, id.bytes, 128);
  return r;
}
// Every rank, with its device current.  Returns the communicator or nullptr (*err = ncclResult_t).
void* lt_nccl_init(const void* id128, int world, int rank, int* err) {
  if (!load()) { if (err) *err = -1; return nullptr; }
  NcclId id;
  memcpy(id.bytes, id128, 128);
  Comm c = nullptr;
  const int r = g_api.CommInitRank(&c, world, id, rank);
  if (err) *err = r;
  return r == 0 ? c : nullptr;
}
int lt_nccl_destroy(void* comm) { return load() ? g_api.CommDestroy(comm) : -1; }
// dtype / op are NCCL's codes (float32 7, float16 6, bfloat16 9, int32 2, int64 4, uint8 1; sum 0, prod 1, max 2, min 3, avg 4).
int lt_nccl_all_reduce(void* comm, const void* send, void* recv, unsigned long long count, int dtype, int op, void* stream) {
  return g_api.AllReduce(send, recv, count, dtype, op, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_all_gather(void* comm, const void* send, void* recv, unsigned long long send_count, int dtype, void* stream) {
  return g_api.AllGather(send, recv, send_count, dtype, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_reduce_scatter(void* comm, const void* send, void* recv, unsigned long long recv_count, int dtype, int op, void* stream) {
  return g_api.ReduceScatter(send, recv, recv_count, dtype, op, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_broadcast(void* comm, const void* send, void* recv, unsigned long long count, int dtype, int root, void* stream) {
  return g_api.Broadcast(send, recv, count, dtype, root, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_send(void* comm, const void* buf, unsigned long long count, int dtype, int peer, void* stream) {
  return g_api.Send(buf, count, dtype, peer, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_recv(void* comm, void* buf, unsigned long long count, int dtype, int peer, void* stream) {
  return g_api.Recv(buf, count, dtype, peer, comm, static_cast<cudaStream_t>(stream));
}
int lt_nccl_group_start() { return load() ? g_api.GroupStart() : -1; }
int lt_nccl_group_end() { return load() ? g_api.GroupEnd() : -1; }

}  // extern "C"
