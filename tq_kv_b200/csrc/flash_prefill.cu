// Causal grouped-query attention for steps that bring many tokens per
// sequence (prompts), bfloat16, on the tensor cores.  A block of 4 warps owns
// 64 consecutive query tokens of one (sequence, q head); it walks the key
// range in tiles of 64 keys that all warps share in shared memory (cp.async,
// two stages), computes S = Q·K^T and O += P·V with mma.sync m16n8k16 and
// keeps a float32 online softmax per query row.  Keys and values come from
// the step's packed rows or from the paged cache; an optional sliding window
// narrows the key range.  Tiles that lie wholly outside a block's range are
// never loaded.
//
// Formulas: src/models/turbo_generic.rs:1620-1631 (see attention.cu).
#include "common.cuh"

#define FP_WARPS 4
#define FP_BM 64
#define FP_BN 64

__device__ __forceinline__ void fp_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fp_ldmatrix_x4(uint32_t* r, const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void fp_ldmatrix_x4_trans(uint32_t* r, const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void fp_cp_async16(void* smem, const void* gmem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void fp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void fp_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t fp_pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct FpSource {
    const bf16* k_packed;      // [T, nkv, hd] or null
    const bf16* v_packed;
    const bf16* k_pages;       // [pages, nkv, page_tokens, hd]
    const bf16* v_pages;
    const int* block_table;
    int table_width;
    int ring_pages;
    int page_tokens;
};

template <int HD>
__global__ void __launch_bounds__(FP_WARPS * 32)
flash_prefill_kernel(const bf16* __restrict__ q, FpSource src, const int* __restrict__ cu_seqlens,
                     const int* __restrict__ start_pos, int n_seqs, int window, float scale_log2,
                     bf16* __restrict__ out, int nh, int nkv) {
    constexpr int ROW = HD * 2 + 16;                 // padded row: ldmatrix without bank conflicts
    constexpr int TILE = FP_BN * ROW;
    constexpr int KS = HD / 16;
    constexpr int NT = HD / 8;
    constexpr int PR = HD / 8;                       // 16-byte pieces per row
    extern __shared__ __align__(16) unsigned char smem[];   // [2 stages][K tile, V tile]

    // which (sequence, 64-token tile) is this block's?
    int b = -1, tile = blockIdx.x;
    for (int i = 0; i < n_seqs; ++i) {
        const int tiles = (cu_seqlens[i + 1] - cu_seqlens[i] + FP_BM - 1) / FP_BM;
        if (tile < tiles) { b = i; break; }
        tile -= tiles;
    }
    if (b < 0) return;
    const int h = blockIdx.y, g = h / (nh / nkv);
    const int tok0 = cu_seqlens[b], len = cu_seqlens[b + 1] - tok0, start = start_pos[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid4 = lane & 3;

    // rows of this lane: local token index i, absolute position p (rows past the end repeat the last row)
    int ri[2], rp[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        int i = tile * FP_BM + warp * 16 + gid + 8 * r;
        ri[r] = i;
        if (i > len - 1) i = len - 1;
        rp[r] = start + i;
    }
    const int p_first = start + tile * FP_BM;
    const int p_last = start + min(len, tile * FP_BM + FP_BM) - 1;
    int j_begin = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    j_begin &= ~(FP_BN - 1);
    const int n_tiles = (p_last - j_begin) / FP_BN + 1;
    const int packed_base = src.k_packed ? tok0 - start : 0;     // key j lives at packed token packed_base + j

    // Q fragments straight from global memory
    uint32_t qf[KS][4];
    {
        const int i0 = min(ri[0], len - 1), i1 = min(ri[1], len - 1);
        const bf16* q0 = q + ((size_t)(tok0 + i0) * nh + h) * HD;
        const bf16* q1 = q + ((size_t)(tok0 + i1) * nh + h) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = ks * 16 + 2 * tid4;
            qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + d);
            qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + d);
            qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + d + 8);
            qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + d + 8);
        }
    }

    auto load_tile = [&](int it) {
        unsigned char* ks_ = smem + (it & 1) * 2 * TILE;
        unsigned char* vs_ = ks_ + TILE;
        const int j0 = j_begin + it * FP_BN;
        for (int p = threadIdx.x; p < FP_BN * PR; p += FP_WARPS * 32) {
            const int key = p / PR, c = p - key * PR;
            int j = j0 + key;
            if (j > p_last) j = p_last;                        // a valid row; masked in S
            size_t row;
            const bf16 *kb, *vb;
            if (src.k_packed) {
                row = ((size_t)(packed_base + j) * nkv + g) * HD;
                kb = src.k_packed; vb = src.v_packed;
            } else {
                int lp = j / src.page_tokens;
                if (src.ring_pages > 0) lp %= src.ring_pages;
                const int page = src.block_table[(size_t)b * src.table_width + lp];
                row = (((size_t)page * nkv + g) * src.page_tokens + (j % src.page_tokens)) * HD;
                kb = src.k_pages; vb = src.v_pages;
            }
            fp_cp_async16(ks_ + key * ROW + c * 16, kb + row + c * 8);
            fp_cp_async16(vs_ + key * ROW + c * 16, vb + row + c * 8);
        }
        fp_commit();
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    load_tile(0);
    for (int it = 0; it < n_tiles; ++it) {
        if (it + 1 < n_tiles) { load_tile(it + 1); fp_wait<1>(); } else { fp_wait<0>(); }
        __syncthreads();
        const unsigned char* ks_ = smem + (it & 1) * 2 * TILE;
        const unsigned char* vs_ = ks_ + TILE;
        const int j0 = j_begin + it * FP_BN;

        float s[FP_BN / 8][4];
#pragma unroll
        for (int n = 0; n < FP_BN / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int n = 0; n < FP_BN / 8; n += 2) {
                uint32_t kb[4];
                fp_ldmatrix_x4(kb, ks_ + ((n + (mat >> 1)) * 8 + r8) * ROW + (2 * ks + (mat & 1)) * 16);
                fp_mma(s[n], qf[ks], kb[0], kb[1]);
                fp_mma(s[n + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // scale and mask: key j is seen by the row at position p iff p - window < j <= p.  Most tiles lie
        // wholly inside every row's range (the same answer for the whole block): they skip the tests.
        float mx[2] = {-INFINITY, -INFINITY};
        const bool inside = j0 + FP_BN - 1 <= p_first && (window <= 0 || j0 > p_last - window);
        if (inside) {
#pragma unroll
            for (int n = 0; n < FP_BN / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = s[n][e] * scale_log2;
                    s[n][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
        } else {
#pragma unroll
            for (int n = 0; n < FP_BN / 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + n * 8 + 2 * tid4 + (e & 1);
                    const int p = rp[e >> 1];
                    const bool seen = j <= p && (window <= 0 || j > p - window);
                    const float v = seen ? s[n][e] * scale_log2 : -INFINITY;
                    s[n][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            // a row may see nothing of this tile (a window that starts later): keep exp2f away from inf - inf
            corr[r] = m_new == -INFINITY ? 1.f : exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int n = 0; n < FP_BN / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mr = m_run[e >> 1];
                const float p = mr == -INFINITY ? 0.f : exp2f(s[n][e] - mr);
                s[n][e] = p;
                rs[e >> 1] += p;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
        // O += P · V, 16 keys per k-step
#pragma unroll
        for (int kk = 0; kk < FP_BN / 16; ++kk) {
            const uint32_t pf[4] = {fp_pack(s[2 * kk][0], s[2 * kk][1]), fp_pack(s[2 * kk][2], s[2 * kk][3]),
                                    fp_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                    fp_pack(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int n = 0; n < NT; n += 2) {
                uint32_t vb[4];
                fp_ldmatrix_x4_trans(vb, vs_ + (kk * 16 + (mat & 1) * 8 + r8) * ROW + (n + (mat >> 1)) * 16);
                fp_mma(o[n], pf, vb[0], vb[1]);
                fp_mma(o[n + 1], pf, vb[2], vb[3]);
            }
        }
        __syncthreads();                                   // all warps are done with this stage
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (ri[r] >= len) continue;
        const float inv = 1.f / l_run[r];
        bf16* orow = out + ((size_t)(tok0 + ri[r]) * nh + h) * HD;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int d = n * 8 + 2 * tid4;
            *reinterpret_cast<__nv_bfloat162*>(orow + d) =
                __floats2bfloat162_rn(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        }
    }
}

template <int HD>
static int launch_flash_prefill(const bf16* q, const FpSource& src, const int* cu_seqlens, const int* start_pos,
                                int n_seqs, int n_tokens, int window, float scale, bf16* out, int nh, int nkv,
                                cudaStream_t stream) {
    constexpr size_t smem = 2 * 2 * FP_BN * (HD * 2 + 16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    // an upper bound on the number of 64-token tiles: every sequence may add one partial tile
    const dim3 grid((n_tokens + FP_BM - 1) / FP_BM + n_seqs, nh);
    flash_prefill_kernel<HD><<<grid, FP_WARPS * 32, smem, stream>>>(q, src, cu_seqlens, start_pos, n_seqs, window,
                                                                   scale * 1.4426950408889634f, out, nh, nkv);
    return tq_launch_status();
}

// Returns cudaErrorNotSupported (801) for head sizes outside {32, 64, 96, 128};
// the caller then uses the general kernel.
TQ_API int tq_flash_prefill(const void* q, const void* k_packed, const void* v_packed, const void* k_pages,
                            const void* v_pages, const int* block_table, int table_width, int ring_pages,
                            int page_tokens, const int* cu_seqlens, const int* start_pos, int n_seqs, int n_tokens,
                            int window, float scale, void* out, int nh, int nkv, int hd, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh > 65535) return (int)cudaErrorNotSupported;
    if (!k_packed && (!k_pages || !block_table || page_tokens <= 0)) return (int)cudaErrorInvalidValue;
    FpSource src{(const bf16*)k_packed, (const bf16*)v_packed, (const bf16*)k_pages, (const bf16*)v_pages,
                 block_table, table_width, ring_pages, page_tokens};
#define TQ_FP(H)                                                                                              \
    case H:                                                                                                   \
        return launch_flash_prefill<H>((const bf16*)q, src, cu_seqlens, start_pos, n_seqs, n_tokens, window, \
                                       scale, (bf16*)out, nh, nkv, stream)
    switch (hd) {
        TQ_FP(32);
        TQ_FP(64);
        TQ_FP(96);
        TQ_FP(128);
        default: return (int)cudaErrorNotSupported;
    }
#undef TQ_FP
}
