// Decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists for hosts of this
// library that cannot call cudaMalloc themselves and cannot let a library do it for them,
// such as a process that was handed a fixed carve-out of device memory by its parent, a
// real-time loop that may not take the allocator's lock, or a plug-in whose host owns every
// allocation.  The regular entry point (ap_attention_tc, mode 1) asks its caller for
// scratch memory for the partial results of the key slices; this variant keeps that
// scratch in a fixed array inside the library instead.
//
// What the caller must know:
//  * Inputs and outputs are still the caller's: q, out, the cache pages and the tables.
//  * The scratch is AP_ATTENTION_STATIC_SCRATCH_FLOATS floats (8 MiB) of device memory that
//    every GPU loading this library holds until the process exits.  The attention library is
//    built once per head size: a process that loads the libraries of several head sizes
//    holds one such array for each of them.
//  * A call needs nsplit * T * num_heads * (head_dim + 2) floats of it when nsplit > 1 and
//    none when nsplit == 1; a call that needs more is refused with AP_ERR_INVALID and a
//    message from ap_last_error(), and nothing is launched.
//  * The first call on a device looks up the array's device address (once per device, with
//    that device current).  Make that first call outside any stream capture.
//  * All calls share the one array, which keeps what the last call left in it.  Nothing in
//    it has to start at zero: every slice of every row is written before it is read.  Two
//    calls that overlap on the GPU (different streams, no ordering) race on it.
//  * No cudaMalloc, cudaFree or other allocating routine runs inside, on any call.
#pragma once
#include <cuda_runtime.h>

#define AP_ATTENTION_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

// Causal attention of T decode rows (one per sequence, row t = sequence t) over paged keys
// and values, bfloat16, for the head size this library was compiled for.
//   q, out       [T, num_heads * head_dim] bfloat16
//   cache        one layer's pages [page][2][num_kv_heads][page_size][head_dim] bfloat16
//   block_table  [T, max_blocks] page ids of each sequence
//   positions    [T] position of each row; it attends to keys 0..position (or the last
//                `window` of them when window > 0)
//   nsplit       key slices per row (>= 1)
// Returns 0, or a status code with the text available from ap_last_error().
int ap_attention_decode_static(const void* q, void* out, const void* cache, const int* block_table,
                               int max_blocks, const int* positions, int T, int num_heads,
                               int num_kv_heads, int head_dim, int page_size, long long page_stride,
                               float scale, int window, int nsplit, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
