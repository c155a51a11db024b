// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference engine; it exists for callers of this
// library that are not allowed to allocate device memory at the time of the call:
//   * code running between cudaStreamBeginCapture and cudaStreamEndCapture of a stream it does
//     not own (cudaMalloc is not permitted during capture),
//   * plug-ins hosted by a runtime that hands out a fixed device arena at start-up and forbids
//     cudaMalloc / cudaFree afterwards (real-time or safety-certified hosts, sandboxes that
//     intercept the allocator), and
//   * callers that hold every byte of the device for weights and KV cache and must not trigger
//     an out-of-memory failure in the middle of a step.
// Such callers still pass their own input and output buffers.  Only the kernel's scratch memory
// (the split-KV partial results of paged attention) is taken from a fixed array inside the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch array, in floats (8 MiB).  Every GPU whose context loads the
// library holds this array until the process exits.
#define POOT_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)

// Paged attention with split-KV, identical in arguments and result to poot_attn_paged() except that
// the caller passes no scratch pointers: the partial results live in the library's own device array.
//
//   need = R * Hq * splits * (D + 2) floats must not exceed POOT_NOALLOC_SCRATCH_FLOATS;
//   a larger request returns cudaErrorInvalidValue (1) and launches nothing.
//
// The call performs no cudaMalloc, cudaFree or any other allocating routine.  The first call on a
// device resolves the array's device address (cudaGetSymbolAddress) and caches it for that device;
// make that first call outside of any stream capture.  Host threads may make their first calls at
// the same time: each resolves the same address and stores the same value.  Head counts that are
// not positive, or query heads that are not a multiple of the K/V heads, return
// cudaErrorInvalidValue (1) like every other bad request.  All calls share the one array, which keeps
// the previous call's contents: the kernels overwrite every partial they later read, so nothing has
// to be cleared, but two calls that run concurrently on the GPU (different streams, or graphs that
// overlap) race on it - serialise them.
int poot_attn_paged_noalloc(const void* q, int q_stride, const void* kpool, const void* vpool,
                            const int* block_tables, int max_blocks, const int* row_seq, const int* row_ctx,
                            void* out, int out_stride, int R, int Hq, int Hkv, int D, float scale, float softcap,
                            int window, int splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
