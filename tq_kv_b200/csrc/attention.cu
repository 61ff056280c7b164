// Grouped-query attention over the keys and values of a step (packed) or of
// the paged cache, for any number of tokens per sequence, with an optional
// sliding window.  One kernel serves prompts (one split) and decoding (the
// key range is cut into splits whose partial results a second kernel merges
// in a fixed order).  Softmax is float32 with a running maximum.
//
// Reference formulas: src/models/turbo_generic.rs:1620-1631 — scores
// q·k / sqrt(head_dim) of q head h against kv head h / n_rep, keys after the
// query masked (-inf), softmax over keys, times V.  The window (not in the
// reference) lets the query at position p see keys max(0, p-window+1) .. p.
#include "common.cuh"

#define ATT_MAX_PAIRS 4   // head_dim <= 256: each lane owns up to 4 pairs of dims

struct KVSource {
    // packed: rows of this step, [T, nkv, hd]; key at position j of row b is token cu[b] + j - start[b]
    const void* k_packed;
    const void* v_packed;
    // paged: [pages, nkv, page_tokens, hd]
    const void* k_pages;
    const void* v_pages;
    const int* block_table;
    int table_width;
    int ring_pages;
    int page_tokens;
};

template <typename TC>
__device__ __forceinline__ void kv_rows(const KVSource& src, int b, int j, int g, int nkv, int hd, int tok0,
                                        const TC*& krow, const TC*& vrow) {
    if (src.k_packed) {
        const size_t r = ((size_t)(tok0 + j) * nkv + g) * hd;
        krow = (const TC*)src.k_packed + r;
        vrow = (const TC*)src.v_packed + r;
    } else {
        int lp = j / src.page_tokens;
        if (src.ring_pages > 0) lp %= src.ring_pages;
        const int page = src.block_table[(size_t)b * src.table_width + lp];
        const size_t r = (((size_t)page * nkv + g) * src.page_tokens + (j % src.page_tokens)) * hd;
        krow = (const TC*)src.k_pages + r;
        vrow = (const TC*)src.v_pages + r;
    }
}

// grid (token, kv head, split); block = n_warps warps, warp w serves q heads
// g*n_rep + w, + n_warps, ...
template <typename TC>
__global__ void attention_kernel(const TC* __restrict__ q, KVSource src, const int* __restrict__ tok_pos,
                                 const int* __restrict__ tok_seq, const int* __restrict__ cu_seqlens,
                                 const int* __restrict__ start_pos, int window, float scale, TC* __restrict__ out,
                                 float* __restrict__ part_acc, float* __restrict__ part_ml, int nh, int nkv, int hd,
                                 int n_splits) {
    extern __shared__ float q_sh[];   // [n_warps][hd]
    const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int n_rep = nh / nkv;
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const int tok0 = src.k_packed ? cu_seqlens[b] - start_pos[b] : 0;
    const int lo_all = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int lo = lo_all, hi = pos + 1;                      // [lo, hi): this block's keys
    if (n_splits > 1) {
        // every token cuts its own key range into n_splits equal parts (multiples of 32 keys)
        const int keys = pos + 1 - lo_all;
        const int split_len = (((keys + n_splits - 1) / n_splits) + 31) & ~31;
        lo = lo_all + split * split_len;
        if (lo + split_len < hi) hi = lo + split_len;
    }
    float* qs = q_sh + warp * hd;
    constexpr int VEC = Vec16<TC>::N;

    for (int hr = warp; hr < n_rep; hr += n_warps) {
        const int h = g * n_rep + hr;
        const TC* qrow = q + ((size_t)t * nh + h) * hd;
        __syncwarp();
        for (int d = lane; d < hd; d += 32) qs[d] = to_f32<TC>(qrow[d]);
        __syncwarp();

        float m = -INFINITY, l = 0.f;
        float acc[2 * ATT_MAX_PAIRS];
#pragma unroll
        for (int i = 0; i < 2 * ATT_MAX_PAIRS; ++i) acc[i] = 0.f;

        for (int base = lo; base < hi; base += 32) {
            const int j = base + lane;
            const bool valid = j < hi;
            const TC *krow = nullptr, *vrow = nullptr;
            float s = -INFINITY;
            if (valid) {
                kv_rows<TC>(src, b, j, g, nkv, hd, tok0, krow, vrow);
                float dot = 0.f;
                for (int d = 0; d < hd; d += VEC) {
                    float kv[VEC];
                    load16_f32<TC>(krow + d, kv);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dot = fmaf(qs[d + e], kv[e], dot);
                }
                s = dot * scale;
            }
            const float m_new = fmaxf(m, warp_max(s));       // finite: lane 0 of a chunk is always valid
            const float p = valid ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);               // exp(-inf) = 0 on the first chunk
            l = l * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < 2 * ATT_MAX_PAIRS; ++i) acc[i] *= corr;
            m = m_new;
            const int n_here = min(32, hi - base);
            for (int jj = 0; jj < n_here; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                const TC* vr = (const TC*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, jj);
#pragma unroll
                for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
                    const int d = 2 * lane + 64 * i;
                    if (d < hd) {
                        const float2 vv = load2_f32<TC>(vr + d);
                        acc[2 * i] = fmaf(pj, vv.x, acc[2 * i]);
                        acc[2 * i + 1] = fmaf(pj, vv.y, acc[2 * i + 1]);
                    }
                }
            }
        }

        if (n_splits == 1) {
            const float inv = 1.f / l;
            TC* o = out + ((size_t)t * nh + h) * hd;
#pragma unroll
            for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
                const int d = 2 * lane + 64 * i;
                if (d < hd) store2_f32<TC>(o + d, acc[2 * i] * inv, acc[2 * i + 1] * inv);
            }
        } else {
            const size_t r = ((size_t)t * nh + h) * n_splits + split;
            float* pa = part_acc + r * hd;
#pragma unroll
            for (int i = 0; i < ATT_MAX_PAIRS; ++i) {
                const int d = 2 * lane + 64 * i;
                if (d < hd) store2_f32<float>(pa + d, acc[2 * i], acc[2 * i + 1]);
            }
            if (lane == 0) { part_ml[2 * r] = m; part_ml[2 * r + 1] = l; }
        }
    }
}

// Merges the splits of one (token, head): grid (token, head), block 128.
// Splits are combined in index order, so the result does not depend on
// scheduling.  An empty split has m = -inf and l = 0 and contributes nothing.
template <typename TC>
__global__ void attention_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                       TC* __restrict__ out, int nh, int hd, int n_splits) {
    const size_t r0 = ((size_t)blockIdx.x * nh + blockIdx.y) * n_splits;
    const int lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch();
    // every warp finds the maximum and the sum for itself, its lanes striding over the splits
    float m = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) m = fmaxf(m, part_ml[2 * (r0 + s)]);
    m = warp_max(m);
    float l = 0.f;
    for (int s = lane; s < n_splits; s += 32) {
        const float ms = part_ml[2 * (r0 + s)];
        if (ms > -INFINITY) l += part_ml[2 * (r0 + s) + 1] * expf(ms - m);
    }
    l = warp_sum(l);
    TC* o = out + ((size_t)blockIdx.x * nh + blockIdx.y) * hd;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float a = 0.f;
        // the loads do not wait for one another: a split without keys is dropped after its load, not around it
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[2 * (r0 + s)];
            const float v = part_acc[(r0 + s) * hd + d];
            a += ms > -INFINITY ? v * expf(ms - m) : 0.f;
        }
        o[d] = from_f32<TC>(a / l);
    }
}

// Scratch needed for n_splits > 1: part_acc float[T*nh*n_splits*hd], part_ml float[T*nh*n_splits*2].
TQ_API int tq_attention(const void* q, int dtype, const void* k_packed, const void* v_packed, const void* k_pages,
                        const void* v_pages, const int* block_table, int table_width, int ring_pages,
                        int page_tokens, const int* tok_pos, const int* tok_seq, const int* cu_seqlens,
                        const int* start_pos, int window, float scale, void* out, float* part_acc, float* part_ml,
                        int n_tokens, int nh, int nkv, int hd, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > 64 * ATT_MAX_PAIRS || hd % 16 || nkv <= 0 || nh % nkv) return (int)cudaErrorInvalidValue;
    if (n_splits < 1 || (n_splits > 1 && (!part_acc || !part_ml))) return (int)cudaErrorInvalidValue;
    if (!k_packed && (!k_pages || !block_table || page_tokens <= 0)) return (int)cudaErrorInvalidValue;
    if (nkv > 65535 || n_splits > 65535) return (int)cudaErrorInvalidValue;
    KVSource src{k_packed, v_packed, k_pages, v_pages, block_table, table_width, ring_pages, page_tokens};
    const int n_rep = nh / nkv;
    const int n_warps = n_rep < 8 ? n_rep : 8;
    const dim3 grid(n_tokens, nkv, n_splits);
    const size_t smem = (size_t)n_warps * hd * sizeof(float);
    if (dtype == TQ_F32)
        attention_kernel<float><<<grid, n_warps * 32, smem, stream>>>(
            (const float*)q, src, tok_pos, tok_seq, cu_seqlens, start_pos, window, scale, (float*)out, part_acc,
            part_ml, nh, nkv, hd, n_splits);
    else if (dtype == TQ_BF16)
        attention_kernel<bf16><<<grid, n_warps * 32, smem, stream>>>(
            (const bf16*)q, src, tok_pos, tok_seq, cu_seqlens, start_pos, window, scale, (bf16*)out, part_acc,
            part_ml, nh, nkv, hd, n_splits);
    else
        return (int)cudaErrorInvalidValue;
    int st = tq_launch_status();
    if (st || n_splits == 1) return st;
    const dim3 mgrid(n_tokens, nh);
    if (dtype == TQ_F32)
        attention_merge_kernel<float><<<mgrid, 128, 0, stream>>>(part_acc, part_ml, (float*)out, nh, hd, n_splits);
    else
        attention_merge_kernel<bf16><<<mgrid, 128, 0, stream>>>(part_acc, part_ml, (bf16*)out, nh, hd, n_splits);
    return tq_launch_status();
}

// The merge step alone, for kernels that write (unnormalised output, max, sum) per split themselves.
TQ_API int tq_attention_merge(const float* part_acc, const float* part_ml, void* out, int dtype, int n_tokens, int nh,
                              int hd, int n_splits, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_splits < 1 || !part_acc || !part_ml) return (int)cudaErrorInvalidValue;
    const dim3 mgrid(n_tokens, nh);
    if (dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_MERGE, attention_merge_kernel<float>, mgrid, dim3(128), 0, stream, part_acc, part_ml,
                             (float*)out, nh, hd, n_splits);
    if (dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_MERGE, attention_merge_kernel<bf16>, mgrid, dim3(128), 0, stream, part_acc, part_ml,
                             (bf16*)out, nh, hd, n_splits);
    return (int)cudaErrorInvalidValue;
}
