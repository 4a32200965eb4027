/* Decode attention for callers that are not allowed to allocate device memory.
 *
 * This entry point has no counterpart in yuzheng310/qwen3-runtime; it exists for the users
 * of this library described below.
 *
 * The ordinary entry point, q3_paged_attention_decode, cuts each sequence's keys into
 * slices and needs scratch memory for the slices' partial results; its caller allocates
 * that scratch.  Some callers cannot do so: a plugin inside a host program that has given
 * all device memory to its own pool and forbids cudaMalloc; a latency-critical loop where
 * the device-wide synchronisation that cudaMalloc and cudaFree imply is not acceptable; a
 * process whose memory budget was fixed at start-up.  For them this variant keeps the
 * scratch in a fixed array inside the library itself.
 *
 *   - The scratch is a file-scope `static __device__` array of Q3_NO_ALLOC_SCRATCH_FLOATS
 *     floats (8 MiB).  Every GPU on which the library is loaded holds it until the process
 *     exits, whether or not this entry point is ever called.
 *   - Limit: num_seqs * nq * num_splits * (D + 1) must not exceed
 *     Q3_NO_ALLOC_SCRATCH_FLOATS (for example 64 sequences x 32 heads x 7 slices at D = 128).
 *     Larger requests are refused with Q3_ERR_SCRATCH_TOO_SMALL and nothing is launched;
 *     q3_no_alloc_last_error() then returns a sentence that says what was asked and what fits.
 *   - It calls no cudaMalloc, cudaFree or any library routine that allocates.  The caller
 *     passes inputs and outputs exactly as for q3_paged_attention_decode, minus the two
 *     scratch pointers.
 *   - The first call on each device looks up the array's device address (once, with that
 *     device current) before launching.  Make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the previous call
 *     left in it.  Nothing in it has to start at zero: every partial result that the merge
 *     step reads was written by the same call (an empty slice writes log-sum-exp = -inf).
 *     Because the array is shared, two calls that overlap on the GPU (different streams,
 *     or different host threads) race on it: callers must order them.
 */
#pragma once
#include <cuda_runtime.h>

#define Q3_NO_ALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define Q3_ERR_SCRATCH_TOO_SMALL 4

#ifdef __cplusplus
extern "C" {
#endif

/* Same arguments and result as q3_paged_attention_decode without mid_o / mid_lse.
 * Returns 0 on success, Q3_ERR_SCRATCH_TOO_SMALL when the request exceeds the fixed
 * scratch, another non-zero code for bad arguments or a failed launch or set-up. */
int q3_paged_attention_decode_no_alloc(const void* q, int q_stride, const void* kpages, const void* vpages,
                                       const int* block_table, int max_pages, const int* kv_lens,
                                       const int* cu_seqlens, const int* seq_list, void* out, int num_seqs, int nq,
                                       int nkv, int D, int ps, float scale, int window, int num_splits,
                                       cudaStream_t stream);

/* Text of the last refusal or set-up failure of the call above on this host thread ("" if none). */
const char* q3_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
