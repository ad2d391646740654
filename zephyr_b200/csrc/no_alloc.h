// zb_paged_decode_no_alloc: decode attention for callers that must not allocate.
//
// This entry point has no counterpart in the reference project.  It exists for hosts that embed
// the kernel library where device allocation is off limits: a plug-in running inside another
// program's memory budget, a real-time loop that may not take the allocator's lock, a process
// whose allocator belongs to a framework the caller cannot reach.  zb_paged_decode needs a
// scratch buffer for the partial results of the context splits, which such a caller could not
// provide; here the scratch is a fixed array that is part of the library image itself.
//
// Limit: the arrival counters and the partial results must fit ZB_NO_ALLOC_SCRATCH_BYTES (4 MiB).
// How much that is depends on how the work is cut, as in zb_paged_decode:
//     split_size > 0 (fixed splits):   n_rows * num_kv_heads * 4 (rounded up to 256)
//                                      + n_rows * num_heads * max_splits * (head_dim + 2) * 4 bytes,
//         for example 31 rows of 16 heads of size 128 at 4,096 tokens of context (16 splits of 256);
//     split_size == 0 (balanced items): the same counters
//                                      + 2 * 256 * (num_heads / num_kv_heads) * (head_dim + 2) * 4 bytes,
//         whatever n_rows and max_splits are: groups of up to 15 query heads at head size 128 fit, a
//         group of 16 does not.
// zb_paged_decode_no_alloc_bytes_needed gives the figure.  A larger problem is refused with
// ZB_ERR_SCRATCH_TOO_SMALL before anything is cleared or launched.
// Every GPU on which the library is loaded holds these 4 MiB until the process exits.
//
// The first call on a device looks up the array's device address (once per device, with that
// device current); make that first call outside any stream capture.  All calls share the one
// array, which keeps whatever the last call left in it.  The arrival counters at its head must be
// zero when the kernel starts, so every call clears them first (a memset on the caller's stream);
// every partial result a call reads it has written itself.  Two calls whose kernels overlap on
// the GPU (different streams, no ordering between them) would overwrite each other's partial
// results: order them, or use zb_paged_decode with separate buffers.
//
// The call itself performs no cudaMalloc, cudaFree or any other allocating routine; inputs and the
// output are the caller's buffers, exactly as for zb_paged_decode.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define ZB_NO_ALLOC_SCRATCH_BYTES (4u << 20)
#define ZB_ERR_SCRATCH_TOO_SMALL 4   /* the problem needs more scratch than the fixed array holds */
#define ZB_ERR_SCRATCH_ADDRESS 5     /* the array's device address could not be looked up */

/* Same arguments as zb_paged_decode without `scratch`.  Returns 0 when both kernels were launched. */
int zb_paged_decode_no_alloc(void* out, const void* q, const void* kv_cache, const int* block_table, int max_blocks,
                             int page_size, int num_pages, int num_rows, const int* rows, int n_rows,
                             const int* row_q_start, const int* row_ctx, int nh, int nkv, int hd, int window,
                             float scale, int split_size, int max_splits, int* status, void* stream);

/* Bytes of scratch a problem needs (compare with ZB_NO_ALLOC_SCRATCH_BYTES before calling); -1 for
   arguments outside the contract. */
long long zb_paged_decode_no_alloc_bytes_needed(int n_rows, int nh, int nkv, int hd, int split_size, int max_splits);

/* A sentence for a return code of zb_paged_decode_no_alloc. */
const char* zb_paged_decode_no_alloc_error(int code);

#ifdef __cplusplus
}
#endif
