// llg_attn_decode_noalloc: decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (MjrTom/daisi-llogos); it exists for this
// library's own users.  Some of them drive the kernels from places where cudaMalloc is not an
// option: a host thread that must never block on the allocator, a plugin that runs inside
// another program's memory budget, a real-time loop that was told "no allocation after start-up".
// The ordinary entry point, llg_attn_decode_simt, asks its caller for scratch memory to hold the
// partial results of the key splits; this one brings its own: a fixed array that is part of the
// library's image on the device.
//
// What the caller must know:
//   * Limit.  n_seqs * n_heads * n_splits * (head_dim + 2) must not exceed
//     LLG_ATTN_NOALLOC_MAX_FLOATS (1,048,576 floats, 4 MiB); larger requests are refused with an
//     error and nothing is launched.  Every GPU that loads the library holds these 4 MiB until
//     the process exits, whether or not this function is ever called.
//   * First call.  The first call on each device looks up the array's device address (with that
//     device current).  Make that first call before any stream capture begins.
//   * No allocation.  The function calls no cudaMalloc, no cudaFree and no library routine that
//     allocates; inputs and outputs remain the caller's.
//   * Sharing.  All calls use the same array.  It keeps whatever the last call left there; that
//     is harmless, because every value a call reads from it was written by that same call
//     (nothing needs to start at zero).  Two calls whose kernels overlap on the GPU (different
//     streams, or different host threads without ordering) race on the array: keep calls ordered.
#pragma once

#include <cuda_runtime.h>

#define LLG_ATTN_NOALLOC_MAX_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Attention of one new token per sequence over the paged cache; same arithmetic and same result
// as llg_attn_decode_simt.  q is [n_seqs][n_heads][head_dim], out is [n_seqs][n_heads * head_dim],
// both of `dtype` (0 float32, 1 bfloat16) like the cache pages [pages][n_kv][64][head_dim].
// len_before[b] is the number of keys of sequence b before this token (its own key already lies
// in the cache at that position).  Returns 0, or non-zero with a message in llg_last_error().
__attribute__((visibility("default")))
int llg_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* page_table,
                            int table_width, int ring_pages, const int* slots, const int* len_before, void* out,
                            int dtype, int n_seqs, int n_heads, int n_kv_heads, int head_dim, int n_splits,
                            float scale, int window, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
