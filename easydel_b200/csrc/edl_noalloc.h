// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference (EasyDeL); it exists for callers of
// this library that are not able to allocate device memory at the point of the call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Upper limits of edl_rmsnorm_bwd_noalloc. Requests beyond them are rejected with an error.
#define EDL_NOALLOC_RMSNORM_MAX_D 8192           /* widest row (elements) */
#define EDL_NOALLOC_RMSNORM_MAX_PARTIALS 160     /* partial weight-gradient rows (one per CTA) */

// RMSNorm backward without any allocation by the library or on its behalf.
//
// Who needs this: a process that has already handed every free byte of device memory to
// something else (a serving engine that sized its KV page pool to the remaining HBM), or a
// loop that must not allocate once it is running because cudaMalloc may synchronise the
// device and its latency is unbounded. The regular entry point, edl_rmsnorm_bwd, asks the
// caller for a scratch buffer of edl_rmsnorm_bwd_workspace(rows, D) floats, which such a
// caller would have to allocate. This one keeps its scratch (the per-CTA partial sums of the
// weight gradient) in a fixed array inside the library instead:
// EDL_NOALLOC_RMSNORM_MAX_PARTIALS x EDL_NOALLOC_RMSNORM_MAX_D floats = 5 MiB, which every
// GPU that loads the library holds until the process exits.
//
// Math and arguments are those of edl_rmsnorm_bwd (bf16 x/w/dy/dres/dx, fp32 rstd and dw):
//   dx = rstd * (g - xhat * mean(g * xhat)) [+ dres],  g = dy * (w + w_offset), xhat = x * rstd
//   dw (+)= sum over rows of dy * xhat          (accumulate != 0 adds to dw)
// x, dy, dx (and dres if given) are [rows, D] contiguous, D a multiple of 8 and at most
// EDL_NOALLOC_RMSNORM_MAX_D; dres and dw may be null; dx may alias dy (or dres). x, w, dy,
// dres and dx must be 16-byte aligned: a misaligned pointer is rejected with an error. The
// caller passes every input and output; nothing is allocated and no allocating routine is
// called.
//
// Set-up: the first call on each device looks up the device address of the scratch array
// (with that device current) and keeps it. Make that first call outside any stream capture.
//
// Sharing: all calls on a device use the same scratch array, and it keeps whatever the
// previous call left in it. Every element that a call reads is written by that same call
// first, so nothing needs to start at zero; but two calls that overlap on the GPU (different
// streams, or different host threads without ordering between their streams) race on it.
// Order such calls on one stream or with events.
//
// Returns 0 on success, non-zero on error (edl_last_error() has the text).
int edl_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                            void* dx, float* dw, int rows, int D, float w_offset, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
