// Allocation-free norm backward.  This entry point has no counterpart in the reference library.
//
// Who needs it: code that drives this library from a place where device memory cannot be requested, for
// example a plugin running inside another framework's memory pool, a host thread that must never block on
// the allocator lock, or a deployment whose memory budget is fixed at start-up.  The regular
// `lt_norm_bwd` needs a caller-provided scratch buffer for the per-CTA partial sums of the weight (and
// bias) gradient, which normally comes from an allocator.  `lt_norm_bwd_noalloc` keeps that scratch in a
// fixed array inside the library image instead, so the caller passes only inputs and outputs.
//
// Cost and limits:
//   * the array is LT_NORM_NOALLOC_SCRATCH_BYTES (about 4.6 MiB) and is held by every GPU that loads the
//     library, from load until the process exits;
//   * D must be a multiple of 8 and at most LT_NORM_NOALLOC_MAX_D; larger rows are rejected with
//     LT_NORM_NOALLOC_ERR_TOO_LARGE and nothing is launched;
//   * the backward pass runs on at most LT_NORM_NOALLOC_MAX_CTAS CTAs (the regular entry point may use more);
//   * the first call on each device looks up the device address of the array (a one-time set-up step);
//     make that first call outside any stream capture;
//   * all calls share the one array.  Its previous contents are never read: each CTA overwrites its own
//     slice before the fold kernel sums the slices, so nothing has to be cleared.  Two calls whose kernels
//     overlap on the GPU (different streams, or concurrent host threads) race on it; keep calls on one
//     device ordered on one stream.
// No cudaMalloc / cudaFree / library allocation happens inside the call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define LT_NORM_NOALLOC_MAX_D 4096
#define LT_NORM_NOALLOC_MAX_CTAS 148
#define LT_NORM_NOALLOC_SCRATCH_BYTES (2 * LT_NORM_NOALLOC_MAX_CTAS * LT_NORM_NOALLOC_MAX_D * 4)
#define LT_NORM_NOALLOC_ERR_TOO_LARGE (-100)
#define LT_NORM_NOALLOC_ERR_SETUP (-101)

// Same math and argument meaning as lt_norm_bwd, minus the two scratch pointers:
//   layer_norm != 0: LayerNorm (mean and db used);  == 0: RMSNorm (mean, db ignored).
//   dy, x, w: bf16 [M, D], [M, D], [D];  mean, rstd: fp32 [M];  dres: optional bf16 [M, D] added to dx.
//   dx: bf16 [M, D];  dw, db: [D], fp32 when grads_fp32 != 0 else bf16; accumulate != 0 adds into them.
// Returns 0, one of the LT_NORM_NOALLOC_ERR_* codes, a negative argument error, or a cudaError_t.
// A required pointer that is null (dy, x, w, rstd, dx, dw; mean and db too for LayerNorm) or a bf16 base that is not
// 16-byte aligned is an argument error (-6): nothing is launched.
int lt_norm_bwd_noalloc(int layer_norm, const void* dy, const void* x, const void* w, const float* mean,
                        const float* rstd, const void* dres, void* dx, void* dw, void* db, int grads_fp32,
                        int accumulate, int M, int D, void* stream);

#ifdef __cplusplus
}
#endif
