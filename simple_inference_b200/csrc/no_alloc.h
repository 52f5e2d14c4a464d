// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (Prathmesh234/simple-inference
// allocates freely through torch); it exists for users of this library.
//
// Who cannot allocate: a program that handed the whole GPU to one pool up front (a
// serving process that sized its cache to all free memory leaves nothing for a later
// cudaMalloc); a latency-critical loop that may not take the allocator's lock or the
// device-wide synchronisation cudaMalloc and cudaFree imply; a host written in another
// language that reaches this library through its C symbols and has no torch allocator
// to borrow scratch from.  si_attn_decode needs scratch for the partial results of its
// key splits and expects the caller to bring it; si_attn_decode_static brings its own.
//
//   * The scratch is a file-scope `static __device__` array of
//     SI_ATTN_STATIC_SCRATCH_FLOATS floats (4 MiB), part of the library image: every
//     GPU that loads the library holds it until the process exits.
//   * A call whose splits need more than that is refused with SI_ERR_TOO_LARGE
//     (see si_attn_decode_scratch_floats for the need of a call); nothing is launched.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
//   * The first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and remembers it; make that
//     first call before any stream capture begins.
//   * All calls share the one array and it keeps the previous call's contents.  Nothing
//     in it needs to start at zero: every partial result that the merge step reads is
//     written earlier in the same call.  Two calls that overlap on the GPU (different
//     streams, or graphs replayed concurrently) race on the array; calls on one stream
//     are safe.
//
// Arguments and result are those of si_attn_decode (attention_mma.cu) without the
// scratch pointer.
#pragma once

#include <cuda_runtime.h>

#define SI_ATTN_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

int si_attn_decode_static(const void* q, int q_stride, const void* pool, int n_pages,
                          const int* block_table, int table_stride, const int* cu_q, const int* positions,
                          const int* single_seqs, int n_single, void* out, int out_stride,
                          int n_q_heads, int n_kv_heads, int page_size, float scale, int window,
                          int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
