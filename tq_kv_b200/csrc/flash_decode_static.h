/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference engine; it exists for
 * hosts that embed these kernels where cudaMalloc is off limits: code that
 * runs inside a region where allocation is forbidden (a real-time loop, a
 * plugin whose host owns all device memory, a process that has handed its
 * whole memory budget to another allocator).  Such a caller passes only its
 * inputs and outputs; the split-key scratch that the ordinary entry point
 * (tq_flash_decode + tq_attention_merge) takes from the caller lives here in
 * a fixed array inside the library instead.
 *
 * Limit: TQ_STATIC_SCRATCH_FLOATS floats (4 MiB).  Every GPU that loads the
 * library holds that array from load until the process exits.  A call needs
 *     n_tokens * n_heads * n_splits * (head_dim + 2)
 * floats when n_splits > 1 (none when n_splits == 1); a call that needs more
 * is refused with TQ_STATIC_TOO_LARGE and launches nothing.
 *
 * The first call on a device looks the array's device address up (no
 * allocation) and keeps it; make that first call outside any stream capture.
 * Two host threads that make their first calls on one device at the same
 * moment both look it up and store the same answer.
 *
 * The kernels start only after everything that precedes them in the stream
 * has completed (no early start under a predecessor's tail, unlike the same
 * kernels inside this library's own decode step), so the caller's earlier
 * kernels may write any of the inputs: positions, table, keys, values, q.
 *
 * All calls share the one array.  Nothing in it has to start at zero: every
 * entry that the merge step reads is written by the same call first.  But two
 * calls whose kernels overlap on the GPU (different streams, or the same
 * call issued from two threads) race on it; keep calls that use splits on
 * one stream, or order them yourself.
 */
#pragma once
#include <cuda_runtime.h>

#define TQ_STATIC_SCRATCH_FLOATS (1u << 20)
#define TQ_STATIC_TOO_LARGE (-2)      /* the call needs more scratch than the library holds */
#define TQ_STATIC_UNSUPPORTED (-3)    /* head size / grouping outside the kernel's reach */

#ifdef __cplusplus
extern "C" {
#endif

/* Attention of n_tokens single decoded tokens over the paged bfloat16 cache.
 * Arguments are those of tq_flash_decode without the scratch pointers: q and
 * out [n_tokens, n_heads * head_dim] bfloat16; k_pages / v_pages
 * [pages, n_kv_heads, page_tokens, head_dim]; block_table int32
 * [rows, table_width]; tok_pos / tok_seq int32 [n_tokens]; window 0 = all
 * keys.  Returns 0, a cudaError_t (> 0), or one of the TQ_STATIC_* codes;
 * tq_flash_decode_static_error() describes the last refusal of this thread. */
int tq_flash_decode_static(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                           int table_width, int ring_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                           int window, float scale, void* out, int n_tokens, int n_heads, int n_kv_heads,
                           int head_dim, int n_splits, cudaStream_t stream);

const char* tq_flash_decode_static_error(void);

#ifdef __cplusplus
}
#endif
