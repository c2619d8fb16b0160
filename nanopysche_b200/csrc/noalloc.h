// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference project (which contains no native code at
// all); it exists for callers of this library that are not allowed to allocate device memory:
// code running while a CUDA stream is being captured, a real-time / latency-critical loop that must
// never enter the allocator, or an embedding host that hands the library a fixed memory budget.
// The regular RMSNorm backward (np_rmsnorm_bwd) needs a scratch buffer for its per-CTA partial sums
// of the weight gradient and expects the caller to provide one; this variant keeps that scratch in a
// fixed, statically sized device array inside the library instead.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the static scratch can serve: cols <= NP_NOALLOC_MAX_COLS (any number of rows).
// The array holds NP_NOALLOC_MAX_PARTS x NP_NOALLOC_MAX_COLS floats (about 4.6 MiB) and every GPU
// that loads the library keeps it resident until the process exits.
#define NP_NOALLOC_MAX_COLS 4096
#define NP_NOALLOC_MAX_PARTS 296

// RMSNorm backward without any allocation.
//   dy, x, dx : bf16 [rows, cols]      w, dw : fp32 [cols]      rstd : fp32 [rows]
//   dres      : optional bf16 [rows, cols] added into dx (nullptr for none)
//   accumulate_dw != 0 : dw += ..., else dw = ...
// Returns 0 on success, 1 for an unsupported shape (cols not a multiple of 8), 3 when cols exceeds
// NP_NOALLOC_MAX_COLS, 4xx/5xx for CUDA set-up / launch errors. It never calls cudaMalloc, cudaFree
// or any allocating library routine.
//
// The first call on a device resolves the device address of the static scratch
// (cudaGetSymbolAddress) - make that first call outside of any stream capture. All calls share the
// one scratch array: two calls whose kernels overlap on the GPU (different streams) race on it, so
// keep calls to this entry point on one stream or order them with events. The scratch keeps the
// previous call's contents; each call overwrites every element it later reads.
int np_rmsnorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* rstd, const void* dres,
                           void* dx, float* dw, int rows, int cols, int accumulate_dw, void* stream);

#ifdef __cplusplus
}
#endif
