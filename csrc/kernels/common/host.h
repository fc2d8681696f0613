// Host-side helpers shared by the kernel launchers: per-device status word, tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda), launch-error plumbing.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lt {

// Device int that kernels write an error code to (0 = ok). One per device, created on first use.
int* device_status_word();

// Number of SMs of the current device (cached per device).
int sm_count();

// Encode a 2-D row-major tensor map. `inner` is the contiguous extent (elements), `outer` the number
// of rows, `row_stride_bytes` the pitch. Returns 0 on success, a CUresult otherwise.
int encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_128b);

// 3-D variant: dims/strides listed innermost first; stride[0] is implied by elem_bytes.
int encode_tmap_3d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2,
                   int swizzle_128b);

// 4-D variant.
int encode_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t d3, uint64_t stride1_bytes, uint64_t stride2_bytes, uint64_t stride3_bytes,
                   uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3, int swizzle_128b);

// Every translation unit with bounded waits registers a function that stores the two wait budgets (SM cycles) into
// its own device globals; lt_set_wait_budget_cycles() calls them all for the current device.
void register_wait_budget_setter(int (*fn)(long long local_cycles, long long peer_cycles));

inline int cuda_ok(cudaError_t e) { return e == cudaSuccess ? 0 : int(e); }

}  // namespace lt

#define LT_RETURN_IF_CUDA(expr)                      \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) return int(_e);           \
  } while (0)

#define LT_LAUNCH_CHECK()                            \
  do {                                               \
    cudaError_t _e = cudaGetLastError();             \
    if (_e != cudaSuccess) return int(_e);           \
  } while (0)
