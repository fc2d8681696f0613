// Host-side helpers: status word, SM count, tensor-map encoding via the driver entry point.
#include "lt_cuda.h"
#include "host.h"

#include <mutex>

#include <vector>

namespace lt {

namespace {
std::vector<int (*)(long long, long long)>& wait_budget_setters() {
  static std::vector<int (*)(long long, long long)> v;   // function-local: safe to use from other units' static initialisers
  return v;
}
}  // namespace

void register_wait_budget_setter(int (*fn)(long long, long long)) { wait_budget_setters().push_back(fn); }

namespace {
constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {nullptr};
int g_sms[kMaxDevices] = {0};
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn get_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

CUtensorMapDataType dtype_of(int elem_bytes) {
  switch (elem_bytes) {
    case 1: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case 2: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case 4: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}
}  // namespace

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev]) return g_status[dev];
  int* p = nullptr;
  if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, 256);
  g_status[dev] = p;
  return p;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sms[dev]) return g_sms[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  g_sms[dev] = n;
  return n;
}

int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_128b) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return int(r);
}

int encode_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                   int swizzle_128b) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return int(r);
}

int encode_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t d3, uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes,
                   uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3, int swizzle_128b) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {stride1_bytes, stride2_bytes, stride3_bytes};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype_of(elem_bytes), 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return int(r);
}

}  // namespace lt

extern "C" {

// Read-and-clear the device status word of the current device. Synchronises the device.
int lt_status_fetch() {
  int* p = lt::device_status_word();
  if (!p) return -1;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

int lt_sm_count() { return lt::sm_count(); }

}  // extern "C"

// Budgets of the bounded waits on the current device, in SM cycles: `local_cycles` for mbarriers and flags written on
// this GPU, `peer_cycles` for flags written by another GPU.  Values <= 0 restore the built-in defaults (about 1.5 s
// and 10 s).  Returns 0 or the first cudaError_t.  Call with no kernel of this library in flight.
extern "C" int lt_set_wait_budget_cycles(long long local_cycles, long long peer_cycles) {
  int rc = 0;
  for (auto fn : lt::wait_budget_setters()) {
    const int r = fn(local_cycles, peer_cycles);
    if (r != 0 && rc == 0) rc = r;
  }
  return rc;
}
