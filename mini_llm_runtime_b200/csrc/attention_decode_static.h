/* Decode attention without any allocation by the caller or by the library.
 *
 * This entry point has no counterpart in the reference project: its kernels always receive a
 * scratch tensor that PyTorch allocates per call (csrc/paged_attention_split_cuda.cu:102-103 there).
 *
 * Who needs it.  Some programs that embed these kernels are not allowed to call cudaMalloc at
 * the point where they decode: a real-time loop that may not touch the allocator once it is
 * running, a plug-in inside a host application that hands it a fixed memory budget, code that runs
 * while a memory pool is frozen.  The ordinary entry point, mlr_attention_decode, makes the caller
 * supply a scratch buffer (float32 partial softmax states) and zeroed counters; here both live in a
 * fixed array that is part of the library image, so the caller passes only inputs and outputs.
 *
 * Limit.  The array holds 4 MiB of partial states and 16,384 counters; every GPU that loads the
 * library keeps it until the process exits.  A call whose rows * heads * max_splits *
 * (head_dim + 2) * 4 bytes exceed mlr_attention_decode_static_capacity(), or with more than
 * 16,384 (row, kv head) pairs, is refused with MLR_TOO_LARGE (-4) and launches nothing.
 *
 * First call.  The first call on each device asks the CUDA runtime for the array's address on
 * that device (cudaGetSymbolAddress, with that device current) and remembers it; make that first
 * call outside any stream capture, and from one thread: the remembered address is not guarded by a
 * lock.  Later calls only enqueue a memset of the counters and the kernel on `stream`.  No call
 * allocates or frees device or host memory.  A call that is refused (any negative code) enqueues
 * nothing.
 *
 * Sharing.  All calls on a device use the same array, which still holds the previous call's
 * contents; the counters are cleared by each call, the states are overwritten before they are
 * read.  Two calls that overlap on the GPU (different streams without ordering) race on it:
 * order them on one stream or with events.
 *
 * Arguments are those of mlr_attention_decode without its `scratch` and `counters`:
 *   q, out        [rows of the step, heads, head_dim] bfloat16
 *   k_pool/v_pool [pages, kv_heads, page_size, head_dim] bfloat16
 *   decode_seg    int32 [rows]: indices into the seg_* arrays of the one-row segments to process
 *   seg_q_start   int32: row of each segment in q/out;  seg_pos0: its position (= keys before it)
 *   block_table   int32 [segments, table_width], page ids of each request
 *   chunk         keys per CTA (multiple of 32); max_splits CTAs per (row, kv head): choose it
 *                 >= ceil(longest context / chunk) for full parallelism; a longer context is still
 *                 computed correctly, its last CTA walking the remaining keys
 * Returns 0, a negative MLR_* code, or a positive cudaError_t.
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long long mlr_attention_decode_static_capacity(void);

int mlr_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                const int* decode_seg, const int* seg_q_start, const int* seg_pos0,
                                const int* block_table, int table_width, int rows, int heads, int kv_heads,
                                int head_dim, int page_size, int window, float scale, int chunk,
                                int max_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
