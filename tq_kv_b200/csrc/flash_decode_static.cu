// tq_flash_decode_static: decode attention with its split scratch in a
// fixed device array of this library, for callers that must not allocate
// (see flash_decode_static.h for who they are, the limit and the sharing
// rules).  It launches the same kernels as the ordinary path — the
// flash-decode kernel and the split merge — and only supplies their scratch.
// Built as a library of its own, so nothing of the ordinary path changes.
#include "flash_decode_static.h"

#include <stdio.h>

#include "attention.cu"        // attention_merge_kernel
#include "flash_decode.cu"     // flash_decode_kernel and its launcher

// The scratch.  In host code this name is only a handle for the runtime's
// symbol lookup, not a device address: it must never be handed to a kernel.
static __device__ __align__(256) float tq_static_scratch[TQ_STATIC_SCRATCH_FLOATS];

#define TQ_MAX_DEVICES 64
static float* g_scratch_addr[TQ_MAX_DEVICES];          // device address of the array, per device, once looked up
static thread_local char g_error[256] = "";

extern "C" __attribute__((visibility("default"))) const char* tq_flash_decode_static_error(void) { return g_error; }

// Device address of the scratch on the current device.  The first call per
// device asks the runtime (cudaGetSymbolAddress, with that device current);
// later calls reuse the answer.  No memory is allocated.
static int scratch_address(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= TQ_MAX_DEVICES) {
        snprintf(g_error, sizeof g_error, "device ordinal %d is beyond the %d this library keeps addresses for", dev,
                 TQ_MAX_DEVICES);
        return (int)cudaErrorInvalidDevice;
    }
    if (!g_scratch_addr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, tq_static_scratch);
        if (e != cudaSuccess) {
            snprintf(g_error, sizeof g_error, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return (int)e;
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

extern "C" __attribute__((visibility("default")))
int tq_flash_decode_static(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                           int table_width, int ring_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                           int window, float scale, void* out, int n_tokens, int n_heads, int n_kv_heads,
                           int head_dim, int n_splits, cudaStream_t stream) {
    g_error[0] = 0;
    if (n_tokens <= 0) return 0;
    if (n_splits < 1 || n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0) {
        snprintf(g_error, sizeof g_error, "sizes must be positive (n_splits %d, heads %d/%d, head_dim %d)", n_splits,
                 n_heads, n_kv_heads, head_dim);
        return (int)cudaErrorInvalidValue;
    }
    float *part_acc = nullptr, *part_ml = nullptr;
    if (n_splits > 1) {
        const unsigned long long rows = (unsigned long long)n_tokens * n_heads * n_splits;
        const unsigned long long need = rows * (unsigned long long)(head_dim + 2);
        if (need > TQ_STATIC_SCRATCH_FLOATS) {
            snprintf(g_error, sizeof g_error,
                     "this call needs %llu floats of scratch (%d tokens x %d heads x %d splits x (%d + 2)); the "
                     "library holds %u", need, n_tokens, n_heads, n_splits, head_dim, TQ_STATIC_SCRATCH_FLOATS);
            return TQ_STATIC_TOO_LARGE;
        }
        float* base = nullptr;
        const int st = scratch_address(&base);
        if (st) return st;
        part_acc = base;
        part_ml = base + rows * head_dim;
    }
    // Without an early start: whatever the caller ran before in this stream (a kernel that writes the positions,
    // the table or many keys) has completed before the first block reads anything.
    int st = flash_decode_launch(q, k_pages, v_pages, block_table, table_width, ring_pages, page_tokens, tok_pos,
                                 tok_seq, window, scale, out, part_acc, part_ml, n_tokens, n_heads, n_kv_heads,
                                 head_dim, n_splits, 0, stream);
    if (st == (int)cudaErrorNotSupported) {
        snprintf(g_error, sizeof g_error,
                 "unsupported shape: head_dim %d (32, 64, 96 or 128), %d q heads per key/value head (at most 16), "
                 "pages of %d tokens (64)", head_dim, n_heads / n_kv_heads, page_tokens);
        return TQ_STATIC_UNSUPPORTED;
    }
    if (st || n_splits == 1) return st;
    return tq_attention_merge(part_acc, part_ml, out, TQ_BF16, n_tokens, n_heads, head_dim, n_splits, stream);
}
