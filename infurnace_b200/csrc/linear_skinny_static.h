// ifb_linear_skinny_static: the few-rows matrix product for callers that must not allocate.
//
// This entry point has no counterpart in tylerguest/infurnace; it exists for users of this library.
//
// Who it is for.  Some programs that want to call this kernel are not in a position to ask the
// CUDA runtime for memory at the moment of the call: a plug-in living inside a host application that
// has already handed the whole device to a memory pool of its own (so a cudaMalloc would fail, or
// would take memory the host believes it owns), or a latency-bound serving loop in which cudaMalloc
// and cudaFree are forbidden because they synchronise the whole device and stall every other stream.
// The ordinary entry point, ifb_linear_skinny, leaves the split-k scratch (partial tiles and
// per-tile counters) to the caller, which in this package means a torch allocation.  This one brings
// its scratch with it: a fixed array that is part of the library's device image.
//
// What it computes.  Exactly what ifb_linear_skinny computes, with the same kernel:
//   out[n, o] = sum_k x[n, k] * w[o, k]                       (epilogue 0)
//   out[n, o] = silu(y[n, o]) * y[n, out_features + o]        (epilogue 1, w has 2*out_features rows)
// x [n_rows, k_dim] and w are bfloat16, 16-byte aligned, k_dim a multiple of 8; out is bfloat16
// (out_dtype 1) or float32 (out_dtype 0).  The caller passes inputs and outputs as before; only the
// scratch arguments are gone.  `splits` CTAs share the k range of each 64-feature tile (1: no scratch
// is touched at all).
//
// Limits.  The scratch holds IFB_STATIC_SCRATCH_FLOATS floats of partial tiles (4 MiB) and
// IFB_STATIC_SCRATCH_COUNTERS tile counters (16 KiB).  Every process that loads the library holds
// that much memory on every GPU it uses, from the moment the library's code is loaded on that GPU
// until the process exits.  A call whose sizes need more than that is refused with
// IFB_ERR_SIZE (2) and launches nothing; ifb_linear_skinny_static_need() tells what a call needs.
//
// Rules of use.
//  * The first call on a device looks up the device address of the scratch array (the array's name
//    is only a host-side handle; the kernel needs the address that cudaGetSymbolAddress returns,
//    with that device current).  Make that first call on each device from ordinary code, before any
//    stream capture is begun.
//  * The entry point calls no cudaMalloc, cudaFree or any allocating library routine.  It enqueues a
//    memset of the counters it is about to use and then the kernel, both on `stream`.
//  * All calls on one device share the one array, and the array keeps whatever the last call left in
//    it.  The counters, which must start at zero, are cleared by every call; the partial tiles are
//    overwritten before they are read.  Two calls that can run at the same time on the GPU (on
//    different streams, or from different threads) race on the array: serialise them.
//
// Returns 0, a positive IFB_ERR_* code when it refuses its arguments, or the negated cudaError_t of
// a failed runtime call.
#pragma once
#include <cuda_runtime.h>

#define IFB_STATIC_SCRATCH_FLOATS (1 << 20)
#define IFB_STATIC_SCRATCH_COUNTERS (1 << 12)

#ifdef __cplusplus
extern "C" {
#endif

int ifb_linear_skinny_static(const void* x, const void* w, void* out, int out_dtype, int n_rows, int out_features,
                             int k_dim, int epilogue, int splits, cudaStream_t stream);

// Floats of partial tiles and counters that a call with these sizes needs (both 0 when splits is 1).
void ifb_linear_skinny_static_need(int n_rows, int out_features, int epilogue, int splits, long long* floats,
                                   long long* counters);

#ifdef __cplusplus
}
#endif
