// Greedy token choice for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (jax-ml/jax-llm-examples); it exists for users
// of this library only.
//
// Who needs it: a host program that has already given the whole device to something else and cannot, or
// must not, call cudaMalloc while it runs.  Examples are an engine whose page pool was sized to take all
// free HBM (a later cudaMalloc fails), a plug-in living inside another framework whose allocator owns the
// device memory, and a latency-critical loop in which an allocation (which may synchronise the device) is
// not acceptable.  jlx_argmax, the ordinary entry point of this library, asks the caller for two scratch
// buffers; such a caller has nowhere to get them from.
//
// What it does: the same two-stage argmax as jlx_argmax (lowest index wins ties, NaNs are skipped), with
// the per-chunk partial results kept in a fixed array that is part of the library image itself.
//
// The price, and the rules that follow from it:
//  * The array is JLX_ARGMAX_NOALLOC_MAX_ROWS * 32 * 8 bytes (64 KiB).  Every GPU on which the library is
//    loaded holds it from load until the process ends, whether or not the function is ever called.
//  * More than JLX_ARGMAX_NOALLOC_MAX_ROWS rows are refused with an error; nothing is launched.
//  * All calls on a device share the one array.  Calls that may overlap on the GPU (different streams,
//    different host threads) race on it and give wrong tokens; order them on one stream.  The array keeps
//    what the last call left, and that is harmless: every slot a call reads it has written itself first,
//    so nothing has to be cleared.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress).  Make that
//    first call once, ordinarily, before any stream capture is started on that device.  Host threads that
//    make their first calls at the same time are safe: each looks the address up and stores the same value.
//  * It calls no cudaMalloc, cudaFree or any allocating library routine.
#pragma once
#include <cuda_runtime.h>

#define JLX_ARGMAX_NOALLOC_MAX_ROWS 256

#ifdef __cplusplus
extern "C" {
#endif

// out[m] = index of the largest of logits[m * ld .. m * ld + V), for m < M.  logits: float32 on the device;
// out: int32 on the device.  Returns 0 when the kernels were launched on `stream`; otherwise non-zero, and
// jlx_last_error() of the same library holds the reason.
int jlx_argmax_noalloc(const float* logits, int M, int V, long long ld, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
