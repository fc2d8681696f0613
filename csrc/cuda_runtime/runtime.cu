// CUDA-side runtime: stream-aware caching device allocator (pluggable into PyTorch), CUDA-graph capture and
// replay, and the NVRTC back end of the JIT (compile a generated fused kernel once, cache, launch).
//
// Reference counterparts: CachingAllocator::allocate_gpu / free lists (src/memory_manager/allocator.cpp:80-124),
// stream-capture graphs whose replay is followed by an eager re-run (src/backend/gpu_native/entrypoint.cu:162-215;
// here a replay is only a replay), and the runtime JIT that shells out to `nvcc` and dlopens the result
// (entrypoint.cu:380-417; here NVRTC in process, no temporary files).
#include "kernels/lt_cuda.h"
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

// ------------------------------------------------------------------ allocator
struct Live {
  size_t size;
  std::vector<cudaStream_t> extra;   // streams other than the allocation stream that used the block (lt_cuda_record_stream)
};
struct Deferred {                    // a freed block that other streams may still be reading
  void* ptr; size_t size; int device; cudaStream_t stream;
  std::vector<cudaEvent_t> events;
};
struct Allocator {
  std::mutex mu;
  // (device, stream) -> size-ordered free blocks.  A block is reused only on the stream it was allocated on, so
  // stream order alone separates its old and new use - unless another stream used it too: those uses are
  // announced with lt_cuda_record_stream, and the block then waits in `deferred` until an event recorded on each
  // of those streams at free time has completed.
  std::map<std::pair<int, cudaStream_t>, std::multimap<size_t, void*>> free_lists;
  std::unordered_map<void*, Live> live;
  std::vector<Deferred> deferred;
  size_t cached = 0, allocated = 0, peak = 0, hits = 0, misses = 0;
  size_t max_cached = 0;  // 0 = unlimited
};
Allocator g_alloc;

bool stream_is_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) { cudaGetLastError(); return false; }
  return st != cudaStreamCaptureStatusNone;
}

// Moves deferred blocks whose events have all completed to the free lists.  Caller holds the lock.
void reap_deferred_locked() {
  for (size_t i = 0; i < g_alloc.deferred.size();) {
    Deferred& d = g_alloc.deferred[i];
    bool done = true;
    for (cudaEvent_t e : d.events)
      if (cudaEventQuery(e) != cudaSuccess) { cudaGetLastError(); done = false; break; }
    if (!done) { ++i; continue; }
    for (cudaEvent_t e : d.events) cudaEventDestroy(e);
    g_alloc.free_lists[{d.device, d.stream}].emplace(d.size, d.ptr);
    g_alloc.deferred[i] = std::move(g_alloc.deferred.back());
    g_alloc.deferred.pop_back();
  }
}

size_t round_size(size_t n) {
  if (n < 512) return 512;
  if (n < (1u << 20)) return (n + 511) & ~size_t(511);
  return (n + (2u << 20) - 1) / (2u << 20) * (2u << 20);
}

void release_cached_locked() {
  for (auto& fl : g_alloc.free_lists)
    for (auto& b : fl.second) cudaFree(b.second);
  g_alloc.free_lists.clear();
  g_alloc.cached = 0;
}

// ------------------------------------------------------------------ NVRTC
typedef int (*nvrtcCreateProgram_t)(void**, const char*, const char*, int, const char* const*, const char* const*);
typedef int (*nvrtcCompileProgram_t)(void*, int, const char* const*);
typedef int (*nvrtcGetSize_t)(void*, size_t*);
typedef int (*nvrtcGetData_t)(void*, char*);
typedef int (*nvrtcDestroyProgram_t)(void**);
struct Nvrtc {
  void* lib = nullptr;
  nvrtcCreateProgram_t create = nullptr;
  nvrtcCompileProgram_t compile = nullptr;
  nvrtcGetSize_t cubin_size = nullptr, log_size = nullptr;
  nvrtcGetData_t cubin = nullptr, log = nullptr;
  nvrtcDestroyProgram_t destroy = nullptr;
  bool ok = false;
};
Nvrtc g_nvrtc;
std::mutex g_jit_mu;
struct JitKernel { cudaLibrary_t lib; cudaKernel_t kernel; int n_inputs; };
std::unordered_map<std::string, int> g_jit_cache;  // source -> handle
std::vector<JitKernel> g_jit_kernels;
std::string g_jit_log;

bool load_nvrtc() {
  if (g_nvrtc.ok) return true;
  const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"};
  for (const char* n : names) {
    g_nvrtc.lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (g_nvrtc.lib) break;
  }
  if (!g_nvrtc.lib) return false;
  g_nvrtc.create = (nvrtcCreateProgram_t)dlsym(g_nvrtc.lib, "nvrtcCreateProgram");
  g_nvrtc.compile = (nvrtcCompileProgram_t)dlsym(g_nvrtc.lib, "nvrtcCompileProgram");
  g_nvrtc.cubin_size = (nvrtcGetSize_t)dlsym(g_nvrtc.lib, "nvrtcGetCUBINSize");
  g_nvrtc.cubin = (nvrtcGetData_t)dlsym(g_nvrtc.lib, "nvrtcGetCUBIN");
  g_nvrtc.log_size = (nvrtcGetSize_t)dlsym(g_nvrtc.lib, "nvrtcGetProgramLogSize");
  g_nvrtc.log = (nvrtcGetData_t)dlsym(g_nvrtc.lib, "nvrtcGetProgramLog");
  g_nvrtc.destroy = (nvrtcDestroyProgram_t)dlsym(g_nvrtc.lib, "nvrtcDestroyProgram");
  g_nvrtc.ok = g_nvrtc.create && g_nvrtc.compile && g_nvrtc.cubin_size && g_nvrtc.cubin && g_nvrtc.destroy;
  return g_nvrtc.ok;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ allocator (PyTorch pluggable-allocator ABI)
void* lt_cuda_alloc(ssize_t size, int device, cudaStream_t stream) {
  if (size <= 0) size = 1;
  const size_t sz = round_size(size_t(size));
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  const bool capturing = stream_is_capturing(stream);
  if (!capturing && !g_alloc.deferred.empty()) reap_deferred_locked();
  auto& fl = g_alloc.free_lists[{device, stream}];
  auto it = fl.lower_bound(sz);
  void* ptr = nullptr;
  size_t got = sz;
  if (it != fl.end() && it->first <= 2 * sz) {
    ptr = it->second;
    got = it->first;
    fl.erase(it);
    g_alloc.cached -= got;
    g_alloc.hits++;
  } else {
    // cudaMalloc is not allowed while the stream records a graph: refuse (the caller sees an out-of-memory error)
    // rather than invalidate the capture.  Warm the cache with one eager run before capturing.
    if (capturing) { g_alloc.misses++; return nullptr; }
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != device) cudaSetDevice(device);
    if (cudaMalloc(&ptr, sz) != cudaSuccess) {
      cudaGetLastError();
      release_cached_locked();
      if (cudaMalloc(&ptr, sz) != cudaSuccess) { cudaGetLastError(); ptr = nullptr; }
    }
    if (prev != device) cudaSetDevice(prev);
    g_alloc.misses++;
    if (!ptr) return nullptr;
  }
  g_alloc.live[ptr] = Live{got, {}};
  g_alloc.allocated += got;
  if (g_alloc.allocated > g_alloc.peak) g_alloc.peak = g_alloc.allocated;
  return ptr;
}
void lt_cuda_free(void* ptr, ssize_t, int device, cudaStream_t stream) {
  if (!ptr) return;
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  auto it = g_alloc.live.find(ptr);
  if (it == g_alloc.live.end()) return;
  const size_t sz = it->second.size;
  std::vector<cudaStream_t> extra = std::move(it->second.extra);
  g_alloc.live.erase(it);
  g_alloc.allocated -= sz;
  const bool capturing = stream_is_capturing(stream);
  if (!capturing && g_alloc.max_cached && g_alloc.cached + sz > g_alloc.max_cached && extra.empty()) {
    cudaFree(ptr);       // implicit device synchronisation: nothing can still be using the block afterwards
    return;
  }
  g_alloc.cached += sz;
  if (!extra.empty() && !capturing) {
    Deferred d{ptr, sz, device, stream, {}};
    for (cudaStream_t s : extra) {
      cudaEvent_t e = nullptr;
      if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess && cudaEventRecord(e, s) == cudaSuccess) d.events.push_back(e);
      else { cudaGetLastError(); if (e) cudaEventDestroy(e); }
    }
    g_alloc.deferred.push_back(std::move(d));
    return;
  }
  g_alloc.free_lists[{device, stream}].emplace(sz, ptr);
}
// Announces that `stream` (not the block's allocation stream) uses the block: when the block is freed it is handed
// out again only after the work queued on `stream` up to that moment has finished.  PyTorch's pluggable-allocator
// binding does not forward tensor.record_stream() to the allocator from Python, so callers that pass temporaries
// to side streams call this (lt.cuda.record_stream); a temporary shared with another stream WITHOUT this call may
// be reused too early.
void lt_cuda_record_stream(void* ptr, cudaStream_t stream) {
  if (!ptr) return;
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  auto it = g_alloc.live.find(ptr);
  if (it == g_alloc.live.end()) return;
  for (cudaStream_t s : it->second.extra) if (s == stream) return;
  it->second.extra.push_back(stream);
}
void lt_cuda_empty_cache() {
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  cudaDeviceSynchronize();
  reap_deferred_locked();
  release_cached_locked();
}
void lt_cuda_set_max_cached(uint64_t bytes) { std::lock_guard<std::mutex> lk(g_alloc.mu); g_alloc.max_cached = bytes; }
// out: {cached, allocated, peak, hits, misses}
void lt_cuda_alloc_stats(uint64_t* out5) {
  std::lock_guard<std::mutex> lk(g_alloc.mu);
  out5[0] = g_alloc.cached; out5[1] = g_alloc.allocated; out5[2] = g_alloc.peak; out5[3] = g_alloc.hits; out5[4] = g_alloc.misses;
}

// ------------------------------------------------------------------ peer memory through CUDA IPC
// A rank exports a device allocation as a 64-byte handle plus the offset of `ptr` inside the allocation that holds it
// (PyTorch sub-allocates its segments); the other processes of the node open the handle and get an address in their
// own address space through which their kernels load from and store to that memory over NVLink.  This is the symmetric
// heap of the fused communication kernels without any framework in between; the handles travel through the process
// group's host-side store.  The reference shares host memory the same way with shm_open (src/distributed/shm_ipc.cpp:71-143).
int lt_ipc_export(void* ptr, void* handle_out, unsigned long long* offset_out) {
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range = nullptr;
  if (!range) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return -1;
    range = reinterpret_cast<RangeFn>(fn);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return -2;
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) { cudaGetLastError(); return int(e); }
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = static_cast<unsigned long long>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return 0;
}
// Returns the peer's `ptr` as an address of this process (base of the mapping + offset), or nullptr (*err = cudaError_t).
// *base_out receives the mapping's base, to be passed to lt_ipc_close.
void* lt_ipc_open(const void* handle, unsigned long long offset, void** base_out, int* err) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { cudaGetLastError(); if (err) *err = int(e); return nullptr; }
  if (base_out) *base_out = base;
  if (err) *err = 0;
  return static_cast<char*>(base) + offset;
}
int lt_ipc_close(void* base) { return int(cudaIpcCloseMemHandle(base)); }

// ------------------------------------------------------------------ CUDA graphs
int lt_graph_begin_capture(void* stream) {
  return int(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
}
// Ends the capture and instantiates; returns a handle (nullptr on failure, *err receives the cudaError_t).
void* lt_graph_end_capture(void* stream, int* err) {
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &g);
  if (e != cudaSuccess || !g) { *err = int(e); return nullptr; }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) { *err = int(e); return nullptr; }
  *err = 0;
  return exec;
}
int lt_graph_launch(void* exec, void* stream) {
  return int(cudaGraphLaunch(static_cast<cudaGraphExec_t>(exec), static_cast<cudaStream_t>(stream)));
}
void lt_graph_destroy(void* exec) { if (exec) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(exec)); }

// ------------------------------------------------------------------ JIT (NVRTC)
// Compiles `source` (must define extern "C" __global__ `kernel_name`) for sm_100a, caches by source text.
// Returns a handle >= 0, or -1 (NVRTC missing), -2 (compile error; see lt_jit_last_log), -3 (load error).
int lt_jit_compile(const char* source, const char* kernel_name, int n_inputs) {
  std::lock_guard<std::mutex> lk(g_jit_mu);
  const std::string key = std::string(kernel_name) + "\n" + source;
  auto it = g_jit_cache.find(key);
  if (it != g_jit_cache.end()) return it->second;
  if (!load_nvrtc()) return -1;
  void* prog = nullptr;
  if (g_nvrtc.create(&prog, source, "lt_jit.cu", 0, nullptr, nullptr) != 0) return -2;
  const char* opts[] = {"--gpu-architecture=sm_100a", "-I/usr/local/cuda/include", "--std=c++17", "-default-device"};
  const int rc = g_nvrtc.compile(prog, 4, opts);
  if (g_nvrtc.log_size && g_nvrtc.log) {
    size_t ls = 0;
    g_nvrtc.log_size(prog, &ls);
    g_jit_log.assign(ls, '\0');
    if (ls) g_nvrtc.log(prog, &g_jit_log[0]);
  }
  if (rc != 0) { g_nvrtc.destroy(&prog); return -2; }
  size_t n = 0;
  g_nvrtc.cubin_size(prog, &n);
  std::vector<char> image(n);
  g_nvrtc.cubin(prog, image.data());
  g_nvrtc.destroy(&prog);
  JitKernel k{};
  if (cudaLibraryLoadData(&k.lib, image.data(), nullptr, nullptr, 0, nullptr, nullptr, 0) != cudaSuccess) { cudaGetLastError(); return -3; }
  if (cudaLibraryGetKernel(&k.kernel, k.lib, kernel_name) != cudaSuccess) { cudaGetLastError(); return -3; }
  k.n_inputs = n_inputs;
  g_jit_kernels.push_back(k);
  const int handle = int(g_jit_kernels.size()) - 1;
  g_jit_cache[key] = handle;
  return handle;
}
int lt_jit_last_log(char* buf, int cap) {
  std::lock_guard<std::mutex> lk(g_jit_mu);
  const int n = int(g_jit_log.size());
  if (cap > 0) { const int c = n < cap - 1 ? n : cap - 1; memcpy(buf, g_jit_log.data(), c); buf[c] = 0; }
  return n;
}
// Launches kernel(in0..in{k-1}, out, n) with a grid-stride geometry.
int lt_jit_launch(int handle, const void* const* inputs, int n_inputs, void* out, long long n, void* stream) {
  JitKernel k;
  {
    std::lock_guard<std::mutex> lk(g_jit_mu);
    if (handle < 0 || handle >= int(g_jit_kernels.size())) return -1;
    k = g_jit_kernels[handle];
  }
  if (n_inputs != k.n_inputs || n_inputs > 16) return -2;
  if (n == 0) return 0;
  const void* in_vals[16];
  void* args[18];
  for (int i = 0; i < n_inputs; ++i) { in_vals[i] = inputs[i]; args[i] = &in_vals[i]; }
  args[n_inputs] = &out;
  args[n_inputs + 1] = &n;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return int(cudaLaunchKernel(reinterpret_cast<const void*>(k.kernel), dim3((unsigned)blocks), dim3(256), args, 0,
                              static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
