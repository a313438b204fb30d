// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists for users of this
// library whose code runs where cudaMalloc is off limits. Typical cases: a serving loop
// that has handed all device memory to its own pools at start-up and treats any later
// allocation as a bug; a host application that loads this library as a plug-in and forbids
// allocation after initialisation; a latency-critical path in which cudaMalloc's implicit
// device synchronisation would stall every stream.
//
// lp_attention_decode_noalloc does what lp_attention_decode does (one new token per
// sequence attends over its paged bf16 cache; the pages are shared out over CTAs whose
// partial results are then merged), but takes no scratch pointer: the partial results go to
// a fixed array that lives inside the library's device image.
//
//  * Limit: the partial results need B * H * num_splits * (head_dim + 2) floats; at most
//    LP_NOALLOC_SCRATCH_FLOATS (4 Mi floats = 16 MiB) are available. A larger request is
//    refused with a message (return -1, text from lp_last_error); nothing is launched.
//  * Cost: every GPU on which the library is loaded holds those 16 MiB until the process
//    exits, whether or not this entry point is ever called.
//  * First call on a device: looks up the array's device address (cudaGetSymbolAddress,
//    with that device current) and remembers it per device. Make that first call outside
//    any stream capture.
//  * The array is shared by all calls and keeps the previous call's contents. Nothing in it
//    has to start at zero: every slot that a call reads was written by that same call.
//    Two calls whose kernels overlap on the GPU (different streams, no ordering) race on
//    it; order them on one stream or with events.
//  * The function calls no cudaMalloc, cudaFree or allocating library routine; inputs and
//    outputs are the caller's.
#pragma once

#include <cuda_runtime.h>

#define LP_NOALLOC_SCRATCH_FLOATS (4ll << 20)

#ifdef __cplusplus
extern "C" {
#endif

// q, out: [B, H, head_dim] bf16; pages: [num_pages, 2, G, 64, head_dim] bf16; page_table: [B, pt_stride]
// int32; kv_len: [B] int32 (lengths including the new token). Returns 0, a cudaError_t, or -1 (refused).
int lp_attention_decode_noalloc(const void* q, void* out, const void* pages, const int* page_table, int pt_stride,
                                const int* kv_len, int B, int H, int G, int hd, int page_size, float scale,
                                int window, int pages_per_split, int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
