// Attention of single decoded tokens over the paged cache (bfloat16), built
// for memory bandwidth: one block per (token, key/value head, split of the
// key range); the q heads that share the key/value head form the rows of one
// 16-row tensor-core tile, so every key and value is read once for all of
// them.  Each of the 4 warps owns every fourth 16- or 32-key chunk of the split and
// streams it global -> shared with cp.async (3 stages per warp, no block
// barrier in the loop), computes S = Q·K^T and O += P·V with mma.sync
// m16n8k16, keeps a float32 online softmax per row, and the warps' states
// are merged through shared memory at the end.  With more than one split the
// block writes (unnormalised output, max, sum) for attention_merge_kernel.
//
// Formulas: src/models/turbo_generic.rs:1620-1631 (see attention.cu).
#include "common.cuh"

#define FD_WARPS 4
#define FD_STAGES 3
#define FD_PAGE 64           // tokens per cache page (checked by the launcher)

__device__ __forceinline__ void fd_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fd_ldmatrix_x4(uint32_t* r, const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fd_ldmatrix_x4_trans(uint32_t* r, const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fd_cp_async16(void* smem, const void* gmem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem));
}
__device__ __forceinline__ void fd_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void fd_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint32_t fd_pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// FD_CHUNK: keys per warp iteration — 16, or 32 for heads of up to 64 dims, whose 16-key chunks would be too small.
template <int HD, int FD_CHUNK>
__global__ void __launch_bounds__(FD_WARPS * 32)
flash_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                    const int* __restrict__ block_table, int table_width, int ring_pages,
                    const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, int window, float scale_log2,
                    bf16* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml, int nh, int nkv,
                    int n_splits) {
    constexpr int ROW = HD * 2 + 16;                       // bytes per key row in shared memory (padded)
    constexpr int TILE = FD_CHUNK * ROW;                   // one K or V chunk
    constexpr int WARP_BYTES = FD_STAGES * 2 * TILE;
    constexpr int KS = HD / 16;                            // k-steps of Q·K^T
    constexpr int NT = HD / 8;                             // n-tiles of P·V
    extern __shared__ __align__(16) unsigned char smem[];
    const int t = blockIdx.x, g = blockIdx.y, split = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid4 = lane & 3;
    const int n_rep = nh / nkv;
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const int lo_all = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    int lo = lo_all, hi = pos + 1;
    if (n_splits > 1) {
        const int keys = pos + 1 - lo_all;
        const int split_len = (((keys + n_splits - 1) / n_splits) + 31) & ~31;
        lo = lo_all + split * split_len;
        if (lo + split_len < hi) hi = lo + split_len;
    }
    const int n_chunks = hi > lo ? (hi - lo + FD_CHUNK - 1) / FD_CHUNK : 0;
    unsigned char* my = smem + warp * WARP_BYTES;
    const int* table = block_table + (size_t)b * table_width;

    // issue the copy of this warp's i-th chunk into stage i % FD_STAGES.  Lane l < FD_CHUNK looks up the row
    // of key l; then consecutive lanes copy consecutive 16-byte pieces of a row, so that every 32-byte
    // sector is asked for once.
    constexpr int PR = HD / 8;                              // 16-byte pieces per row
    auto issue = [&](int i) {
        const int chunk = warp + i * FD_WARPS;
        if (chunk < n_chunks) {
            int j = lo + chunk * FD_CHUNK + (lane & (FD_CHUNK - 1));
            if (j >= hi) j = hi - 1;                       // a valid address; the score is masked
            int lp = j / FD_PAGE;
            if (ring_pages > 0) lp %= ring_pages;
            const unsigned long long my_row = (((unsigned long long)table[lp] * nkv + g) * FD_PAGE + (j % FD_PAGE)) * HD;
            unsigned char* ks_ = my + (i % FD_STAGES) * 2 * TILE;
            unsigned char* vs_ = ks_ + TILE;
#pragma unroll
            for (int it = 0; it < FD_CHUNK * PR / 32; ++it) {
                const int p = lane + 32 * it;
                const int key = p / PR, c = p - key * PR;
                const unsigned long long row = __shfl_sync(0xffffffffu, my_row, key);
                fd_cp_async16(ks_ + key * ROW + c * 16, k_pages + row + c * 8);
                fd_cp_async16(vs_ + key * ROW + c * 16, v_pages + row + c * 8);
            }
        }
        fd_commit();                                       // one group per turn, empty or not
    };

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f; }

    const int my_chunks = n_chunks > warp ? (n_chunks - warp + FD_WARPS - 1) / FD_WARPS : 0;
    // Of this step's inputs only q and the newest key (position pos, written by the kernel before) depend on
    // the predecessor; the positions and tables were copied in before the step's first kernel.  A block whose
    // keys are all older starts its copies before it waits.  (Were there earlier tokens of the same sequence
    // in this step, their keys would be new too: then the token is not its sequence's first row.)
    const bool old_keys_only = hi <= pos && (t == 0 || tok_seq[t - 1] != b);
    if (old_keys_only) {
#pragma unroll
        for (int i = 0; i < FD_STAGES - 1; ++i) issue(i);
    }
    // No pdl_launch(): a kernel let in while this one streams the cache only gets in its way (measured: the
    // step is 2 to 4 % slower at batch 8 and 64); the next kernel starts when this one has ended.
    pdl_wait();
    if (!old_keys_only) {
#pragma unroll
        for (int i = 0; i < FD_STAGES - 1; ++i) issue(i);
    }

    // Q fragments: rows = q heads of this group (rows >= n_rep are zero)
    uint32_t qf[KS][4];
    {
        const bf16* q0 = q + ((size_t)t * nh + (size_t)g * n_rep) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int d = ks * 16 + 2 * tid4;
            qf[ks][0] = gid < n_rep ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)gid * HD + d) : 0u;
            qf[ks][1] = gid + 8 < n_rep ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(gid + 8) * HD + d) : 0u;
            qf[ks][2] = gid < n_rep ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)gid * HD + d + 8) : 0u;
            qf[ks][3] = gid + 8 < n_rep ? *reinterpret_cast<const uint32_t*>(q0 + (size_t)(gid + 8) * HD + d + 8) : 0u;
        }
    }

    for (int i = 0; i < my_chunks; ++i) {
        issue(i + FD_STAGES - 1);
        fd_wait<FD_STAGES - 1>();                          // chunk i has landed
        __syncwarp();
        const unsigned char* ks_ = my + (i % FD_STAGES) * 2 * TILE;
        const unsigned char* vs_ = ks_ + TILE;
        const int j0 = lo + (warp + i * FD_WARPS) * FD_CHUNK;

        // S[16 heads x FD_CHUNK keys] = Q · K^T
        constexpr int ST = FD_CHUNK / 8;                   // 8-key tiles of S
        float s[ST][4];
#pragma unroll
        for (int n = 0; n < ST; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
            for (int n = 0; n < ST; n += 2) {
                uint32_t kb[4];
                const int mat = lane >> 3, r = lane & 7;
                fd_ldmatrix_x4(kb, ks_ + ((n + (mat >> 1)) * 8 + r) * ROW + (2 * ks + (mat & 1)) * 16);
                fd_mma(s[n], qf[ks], kb[0], kb[1]);
                fd_mma(s[n + 1], qf[ks], kb[2], kb[3]);
            }
        }
        // scale, mask keys beyond the range, online softmax (rows gid and gid + 8)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < ST; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = j0 + nt * 8 + 2 * tid4 + (e & 1);
                const float v = j < hi ? s[nt][e] * scale_log2 : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);       // finite: key j0 is always in range
            corr[r] = exp2f(m_run[r] - m_new);
            m_run[r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < ST; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = exp2f(s[nt][e] - m_run[e >> 1]);
                s[nt][e] = p;
                rs[e >> 1] += p;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * corr[r] + rs[r];
        }
        // O = O * corr + P · V, 16 keys per k-step
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            o[n][0] *= corr[0]; o[n][1] *= corr[0];
            o[n][2] *= corr[1]; o[n][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < FD_CHUNK / 16; ++kk) {
            const uint32_t pf[4] = {fd_pack(s[2 * kk][0], s[2 * kk][1]), fd_pack(s[2 * kk][2], s[2 * kk][3]),
                                    fd_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]),
                                    fd_pack(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int n = 0; n < NT; n += 2) {
                uint32_t vb[4];
                const int mat = lane >> 3, r = lane & 7;
                fd_ldmatrix_x4_trans(vb, vs_ + (kk * 16 + (mat & 1) * 8 + r) * ROW + (n + (mat >> 1)) * 16);
                fd_mma(o[n], pf, vb[0], vb[1]);
                fd_mma(o[n + 1], pf, vb[2], vb[3]);
            }
        }
        __syncwarp();                                      // the stage may be overwritten by the next issue
    }
    fd_wait<0>();
    __syncthreads();

    // merge the warps: shared memory now holds [warp][16 rows][HD + 2] floats (output, max, sum)
    float* ms = reinterpret_cast<float*>(smem);
    constexpr int RS = HD + 2;
    {
        float* mine = ms + (size_t)warp * 16 * RS;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int d = n * 8 + 2 * tid4;
            mine[gid * RS + d] = o[n][0];
            mine[gid * RS + d + 1] = o[n][1];
            mine[(gid + 8) * RS + d] = o[n][2];
            mine[(gid + 8) * RS + d + 1] = o[n][3];
        }
        if (tid4 == 0) {
            mine[gid * RS + HD] = m_run[0];
            mine[gid * RS + HD + 1] = l_run[0];
            mine[(gid + 8) * RS + HD] = m_run[1];
            mine[(gid + 8) * RS + HD + 1] = l_run[1];
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_rep * HD; e += blockDim.x) {
        const int r = e / HD, d = e - r * HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < FD_WARPS; ++w) m = fmaxf(m, ms[((size_t)w * 16 + r) * RS + HD]);
        float l = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < FD_WARPS; ++w) {
            const float* row = ms + ((size_t)w * 16 + r) * RS;
            if (row[HD] > -INFINITY) {
                const float f = exp2f(row[HD] - m);
                l += row[HD + 1] * f;
                a += row[d] * f;
            }
        }
        const int h = g * n_rep + r;
        if (n_splits == 1) {
            out[((size_t)t * nh + h) * HD + d] = __float2bfloat16_rn(a / l);
        } else {
            const size_t pr = ((size_t)t * nh + h) * n_splits + split;
            part_acc[pr * HD + d] = a;
            if (d == 0) {
                part_ml[2 * pr] = m * 0.6931471805599453f;   // back to natural-log units for the merge kernel
                part_ml[2 * pr + 1] = l;
            }
        }
    }
}

template <int HD>
static int launch_flash_decode(const bf16* q, const bf16* kp, const bf16* vp, const int* table, int table_width,
                               int ring_pages, const int* tok_pos, const int* tok_seq, int window, float scale,
                               bf16* out, float* part_acc, float* part_ml, int n_tokens, int nh, int nkv, int n_splits,
                               int pdl_family, cudaStream_t stream) {
    constexpr int ROW = HD * 2 + 16;
    constexpr int FD_CHUNK = HD <= 64 ? 32 : 16;
    constexpr size_t stage_bytes = (size_t)FD_WARPS * FD_STAGES * 2 * FD_CHUNK * ROW;
    constexpr size_t merge_bytes = (size_t)FD_WARPS * 16 * (HD + 2) * sizeof(float);
    constexpr size_t smem = stage_bytes > merge_bytes ? stage_bytes : merge_bytes;
    static bool configured[64] = {false};         // per device: the attribute belongs to the device's copy of the kernel
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(flash_decode_kernel<HD, FD_CHUNK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const dim3 grid(n_tokens, nkv, n_splits);
    return tq_launch_pdl(pdl_family, flash_decode_kernel<HD, FD_CHUNK>, grid, dim3(FD_WARPS * 32), smem, stream, q, kp, vp, table,
                         table_width, ring_pages, tok_pos, tok_seq, window, scale * 1.4426950408889634f, out, part_acc,
                         part_ml, nh, nkv, n_splits);
}

// Returns cudaErrorNotSupported (801) for shapes outside this kernel's reach
// (head_dim not in {32, 64, 96, 128}, more than 16 q heads per key/value
// head, pages of another size); the caller then uses the general kernel.
//
// `early_start`: launch the kernel so that it may begin while its predecessor in the stream still runs
// (programmatic dependent launch).  Its blocks then read the positions, the block table and every key older than
// the token's own before the predecessor has ended; that is right only if the predecessor writes nothing but q
// and each token's newest key, as the kernels of a decode step do.  With 0 the kernel starts after everything
// before it in the stream has completed, whatever that was.
static int flash_decode_launch(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                               int table_width, int ring_pages, int page_tokens, const int* tok_pos,
                               const int* tok_seq, int window, float scale, void* out, float* part_acc,
                               float* part_ml, int n_tokens, int nh, int nkv, int hd, int n_splits, int early_start,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16 || page_tokens != FD_PAGE || nkv > 65535 || n_splits > 65535)
        return (int)cudaErrorNotSupported;
    if (n_splits < 1 || (n_splits > 1 && (!part_acc || !part_ml))) return (int)cudaErrorInvalidValue;
#define TQ_FD(H)                                                                                                  \
    case H:                                                                                                       \
        return launch_flash_decode<H>((const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table,   \
                                      table_width, ring_pages, tok_pos, tok_seq, window, scale, (bf16*)out,      \
                                      part_acc, part_ml, n_tokens, nh, nkv, n_splits,                \
                                      early_start ? TQ_PDL_FLASH_DECODE : 0, stream)
    switch (hd) {
        TQ_FD(32);
        TQ_FD(64);
        TQ_FD(96);
        TQ_FD(128);
        default: return (int)cudaErrorNotSupported;
    }
#undef TQ_FD
}

TQ_API int tq_flash_decode(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                           int table_width, int ring_pages, int page_tokens, const int* tok_pos, const int* tok_seq,
                           int window, float scale, void* out, float* part_acc, float* part_ml, int n_tokens, int nh,
                           int nkv, int hd, int n_splits, cudaStream_t stream) {
    return flash_decode_launch(q, k_pages, v_pages, block_table, table_width, ring_pages, page_tokens, tok_pos, tok_seq,
                               window, scale, out, part_acc, part_ml, n_tokens, nh, nkv, hd, n_splits, 1, stream);
}
