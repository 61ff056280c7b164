// Causal grouped-query attention for prompts on the tcgen05 tensor cores.
//
// A block owns 128 consecutive query tokens of one (sequence, q head) and walks
// the keys in tiles of 64.  Per tile:
//   S  = Q · K^T      tcgen05.mma, Q and K tiles K-major in shared memory (TMA,
//                     128-byte swizzle), S[128 x 64] float32 in TMEM; two S
//                     buffers, so the next tile's product is issued while this
//                     tile's softmax runs;
//   softmax           four warps, one query row per thread (TMEM lane = row, so
//                     the row maximum and sum need no shuffles), float32; P goes
//                     back into TMEM as bfloat16, over the scores it came from
//                     (tcgen05.st; a 32-bit column holds two neighbouring keys);
//   O += P · V        tcgen05.mma with P as the A operand from TMEM and V as an
//                     MN-major operand from shared memory (the V tile is
//                     [keys][head_dim] as it lies in memory), accumulated in TMEM
//                     over all tiles and read once at the end.
// P and O are scaled against a reference maximum per row that moves only when
// the row's maximum has grown by more than 2^8; then the warp multiplies its
// rows of O in TMEM (tcgen05.ld / st) and the running sums by the same factor.
// The result is the same softmax (any reference gives the same quotient); the
// exponentials stay below 2^8.
// Roles: warp 0 lane 0 issues TMA loads (Q once, K/V tiles through two stages),
// warp 1 lane 0 issues the MMAs, warps 2..5 do the softmax and the final store.
// A block takes 96 KB of shared memory and half an SM's TMEM: two blocks share
// an SM, and one's tensor-core work runs under the other's softmax.  Blocks
// with the most key tiles start first.  Keys and values come from the step's
// packed rows (PAGED = false) or from the paged cache (one 64-token page per
// tile).  An optional sliding window narrows the key range; tiles outside a
// block's range are never loaded.  All mbarrier waits are bounded (see
// gemm_tc.cu).
//
// Order between the threads, beyond the producer/consumer pairs: the MMA
// thread waits for the P·V of the tile before (p_empty) before it issues the
// Q·K^T of the tile after, which writes over that tile's P; a softmax thread
// waits for the phase of p_full before its own before it arrives again (it may
// be a whole tile ahead of the slowest thread, and a second arrival in the
// same phase would stand in for the slow thread's first); the end of the last
// P·V has a barrier of its own (o_done), since the softmax threads follow
// p_empty only when they rescale O and a wait by parity cannot tell a phase
// that is two behind from one that is done.  Two load tests guard this.
//
// Formulas: src/models/turbo_generic.rs:1620-1631 (see attention.cu).
#include <cuda.h>

#include "common.cuh"

#define FT_BM 128
#define FT_BN 64
#define FT_THREADS 192
#define FT_SUB_BYTES (128 * 128)          // a [128 rows x 64 bf16] sub-tile (Q)
#define FT_KV_SUB_BYTES (FT_BN * 128)     // a [64 keys x 64 bf16] sub-tile (K, V)
#define FT_WAIT_CYCLES (4000000000ll)

__device__ __forceinline__ uint32_t ft_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool ft_wait(uint32_t bar, uint32_t parity, bool backoff = false) {
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (backoff) __nanosleep(20);
        if ((i & 255u) == 0 && clock64() - t0 > FT_WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void ft_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ft_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ft_tma(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void ft_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void ft_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
// the same with the A operand in tensor memory (lane = row, a 32-bit column holds two neighbouring bfloat16 of K)
__device__ __forceinline__ void ft_mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void ft_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void ft_ld32_issue(uint32_t taddr, float* v) {   // the caller waits (ft_ld_wait)
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void ft_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// 2^x of the special-function unit (2 ulp; 2^-inf = 0): the probabilities are rounded to bfloat16 anyway
__device__ __forceinline__ float ft_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void ft_st32(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t ft_desc_k(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand, 128-byte swizzle: a row holds 64 MN elements of one k; 8 k-rows form a 1024-byte group
// (stride byte offset); the next 64 MN elements lie `mn_stride` bytes further (leading byte offset)
__device__ __forceinline__ uint64_t ft_desc_mn(uint32_t saddr, uint32_t mn_stride) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((mn_stride >> 4) & 0x3FFF) << 16) |
           ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

template <int HD, bool PAGED>
__global__ void __launch_bounds__(FT_THREADS, 2)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int table_width,
                        int ring_pages, const int* __restrict__ cu_seqlens, const int* __restrict__ start_pos,
                        int n_seqs, int window, float scale_log2, bf16* __restrict__ out, int nh, int nkv,
                        int* __restrict__ status) {
    constexpr int SUBS = HD / 64;                          // 64-column sub-tiles of a Q, K or V tile
    constexpr int Q_BYTES = SUBS * FT_SUB_BYTES;
    constexpr int KV_BYTES = SUBS * FT_KV_SUB_BYTES;       // a K or V tile of 64 keys
    // 1024-byte alignment (the swizzle's period) is asked of the launch, not bought with slack: two blocks
    // must fit an SM.  A base that is not aligned all the same is reported through *status, nothing runs.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if (reinterpret_cast<uintptr_t>(smem_raw) & 1023) {
        if (threadIdx.x == 0 && status) atomicOr(status, 8);
        return;
    }
    unsigned char* q_s = smem_raw;
    unsigned char* k_s = q_s + Q_BYTES;                    // [2 stages]
    unsigned char* v_s = k_s + 2 * KV_BYTES;               // [2 stages]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * KV_BYTES);
    uint64_t* q_full = bars;
    uint64_t* k_full = bars + 1;                           // [2]  K and V have rings of their own: a K stage is
    uint64_t* k_empty = bars + 3;                          // [2]  free as soon as its Q·K^T is done, long before
    uint64_t* v_full = bars + 5;                           // [2]  the tile's P·V, so the load of the tile after
    uint64_t* v_empty = bars + 7;                          // [2]  next has a whole iteration to arrive
    uint64_t* s_full = bars + 9;                           // [2]
    uint64_t* p_full = bars + 11;                          // 128 arrivals (softmax threads)
    uint64_t* p_empty = bars + 12;                         // the P·V of a tile is done: O may be touched
    uint64_t* o_done = bars + 13;                          // once: the last P·V is done, O is final
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile uint32_t* failed = tmem_slot + 1;

    // which (sequence, 128-token tile) is this block's?  Later tiles of a sequence have more keys to walk:
    // the tiles are walked backwards, and the heads are the grid's fast dimension, so that the heaviest tiles
    // of ALL heads start first and the lightest fill the slots that fall free at the end.  (With the tiles
    // as the fast dimension the last heads' heavy tiles started late: 63.5 us for one prompt of 2,048 tokens
    // and 28 heads of 128, where the longest block alone takes about 45.)
    int b = -1, tile = (int)gridDim.y - 1 - (int)blockIdx.y;
    for (int i = 0; i < n_seqs; ++i) {
        const int tiles = (cu_seqlens[i + 1] - cu_seqlens[i] + FT_BM - 1) / FT_BM;
        if (tile < tiles) { b = i; break; }
        tile -= tiles;
    }
    if (b < 0) return;
    const int h = blockIdx.x, g = h / (nh / nkv);
    const int tok0 = cu_seqlens[b], len = cu_seqlens[b + 1] - tok0, start = start_pos[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p_first = start + tile * FT_BM;
    const int p_last = start + min(len, tile * FT_BM + FT_BM) - 1;
    int j_begin = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    j_begin &= ~(FT_BN - 1);
    const int n_tiles = (p_last - j_begin) / FT_BN + 1;

    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(q_full)));
        for (int s = 0; s < 2; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(&k_full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(&k_empty[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(&v_full[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(&v_empty[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(&s_full[s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 128;\n" ::"r"(ft_smem(p_full)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(p_empty)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ft_smem(o_done)));
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(ft_smem(tmem_slot)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_s = *tmem_slot;                    // S: two buffers of 64 columns
    const uint32_t tmem_o = tmem_s + 128;                  // O: columns 128..128+HD, accumulated over the tiles
    // Programmatic dependent launch (common.cuh): q, k and v come from the kernel before; the step's lengths
    // and tables, read above, were copied in before its first kernel.
    pdl_wait();
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer ----
            ft_expect(ft_smem(q_full), Q_BYTES);
            for (int sub = 0; sub < SUBS; ++sub)
                ft_tma(ft_smem(q_s + sub * FT_SUB_BYTES), &map_q, h * HD + sub * 64, tok0 + tile * FT_BM, ft_smem(q_full));
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it & 1;
                const int j0 = j_begin + it * FT_BN;
                int row;
                if (PAGED) {
                    int lp = j0 / 64;
                    if (ring_pages > 0) lp %= ring_pages;
                    row = (block_table[(size_t)b * table_width + lp] * nkv + g) * 64;
                } else {
                    row = tok0 - start + j0;                 // key j lives at packed token tok0 - start + j
                }
                const int col = PAGED ? 0 : g * HD;
                if (!ft_wait(ft_smem(&k_empty[s]), ((it >> 1) & 1) ^ 1)) { *failed = 1; break; }
                ft_expect(ft_smem(&k_full[s]), KV_BYTES);
                for (int sub = 0; sub < SUBS; ++sub)
                    ft_tma(ft_smem(k_s + s * KV_BYTES + sub * FT_KV_SUB_BYTES), &map_k, col + sub * 64, row,
                           ft_smem(&k_full[s]));
                if (!ft_wait(ft_smem(&v_empty[s]), ((it >> 1) & 1) ^ 1)) { *failed = 1; break; }
                ft_expect(ft_smem(&v_full[s]), KV_BYTES);
                for (int sub = 0; sub < SUBS; ++sub)
                    ft_tma(ft_smem(v_s + s * KV_BYTES + sub * FT_KV_SUB_BYTES), &map_v, col + sub * 64, row,
                           ft_smem(&v_full[s]));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FT_BN >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) /* B is MN-major */ |
                                     ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(FT_BM >> 4) << 24);
            bool ok = ft_wait(ft_smem(q_full), 0);
            if (!ok) *failed = 1;
            const uint32_t qa = ft_smem(q_s);
            auto issue_qk = [&](int it) -> bool {            // S[it & 1] = Q · K(it)^T over head_dim
                const int s = it & 1;
                if (!ft_wait(ft_smem(&k_full[s]), (it >> 1) & 1)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t ka = ft_smem(k_s + s * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    ft_mma(tmem_s + s * FT_BN, ft_desc_k(qa + (ks >> 2) * FT_SUB_BYTES + (ks & 3) * 32),
                           ft_desc_k(ka + (ks >> 2) * FT_KV_SUB_BYTES + (ks & 3) * 32), idesc_s, ks > 0 ? 1u : 0u);
                ft_commit(ft_smem(&k_empty[s]));
                ft_commit(ft_smem(&s_full[s]));
                return true;
            };
            if (ok && !issue_qk(0)) { *failed = 1; ok = false; }
            for (int it = 0; it < n_tiles && ok; ++it) {
                const int s = it & 1;
                // The next tile's scores are computed while the softmax threads work on this one.  They go
                // into the buffer that holds the P of the tile before, which that tile's P·V reads as its A
                // operand from tensor memory; nothing documented orders a later MMA's writes behind an earlier
                // MMA's operand reads there, so that P·V has to be complete first.  The same wait keeps the
                // softmax threads within one phase of p_empty, which their wait by parity (when they rescale O)
                // relies on.
                if (it > 0 && !ft_wait(ft_smem(p_empty), (it - 1) & 1)) { *failed = 1; ok = false; break; }
                if (it + 1 < n_tiles && !issue_qk(it + 1)) { *failed = 1; ok = false; break; }
                if (!ft_wait(ft_smem(&v_full[s]), (it >> 1) & 1) || !ft_wait(ft_smem(p_full), it & 1)) {
                    *failed = 1; ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t va = ft_smem(v_s + s * KV_BYTES);
#pragma unroll
                for (int ks = 0; ks < FT_BN / 16; ++ks)      // O += P · V over the tile's 64 keys; P sits where S was
                    ft_mma_ts(tmem_o, tmem_s + s * FT_BN + ks * 8, ft_desc_mn(va + ks * 2048, FT_KV_SUB_BYTES),
                              idesc_o, (it > 0 || ks > 0) ? 1u : 0u);
                ft_commit(ft_smem(&v_empty[s]));             // the stage is free once these MMAs are done
                ft_commit(ft_smem(p_empty));
                if (it == n_tiles - 1) ft_commit(ft_smem(o_done));
            }
        }
    } else {
        // ---- softmax and the final store: thread = query row.  O stays in TMEM; it is accumulated against a
        // reference maximum that only moves when a row's maximum has grown by more than 2^8, in which case the
        // warp rescales its rows of O (and the running sums) — rare after the first tiles. ----
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                   // row of the tile = TMEM lane
        const int i_row = tile * FT_BM + r;                  // token index within the sequence
        const int p_row = start + min(i_row, len - 1);       // rows past the end repeat the last row (never stored)
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        float m_ref = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int it = 0; it < n_tiles && ok; ++it) {
            const int j0 = j_begin + it * FT_BN;
            if (!ft_wait(ft_smem(&s_full[it & 1]), (it >> 1) & 1, true)) { *failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t s_addr = tmem_s + (it & 1) * FT_BN + lane_addr;
            // key j is seen iff p_row - window < j <= p_row; most tiles lie inside every row's range
            const int j_hi = p_row, j_lo = window > 0 ? p_row - window + 1 : 0;
            const bool inside = j0 + FT_BN - 1 <= p_first && (window <= 0 || j0 > p_last - window);
            float sv[FT_BN];                                  // the row's scores of this tile
#pragma unroll
            for (int c = 0; c < FT_BN; c += 32) ft_ld32_issue(s_addr + c, sv + c);
            ft_ld_wait();
            if (!inside) {
#pragma unroll
                for (int j = 0; j < FT_BN; ++j) {
                    const int key = j0 + j;
                    if (key < j_lo || key > j_hi) sv[j] = -INFINITY;     // a masked key: 2^-inf = 0 below
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};    // four chains instead of one of 64
#pragma unroll
            for (int j = 0; j < FT_BN; j += 4) {
                mx4[0] = fmaxf(mx4[0], sv[j]);
                mx4[1] = fmaxf(mx4[1], sv[j + 1]);
                mx4[2] = fmaxf(mx4[2], sv[j + 2]);
                mx4[3] = fmaxf(mx4[3], sv[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_tile = mx * scale_log2;
            const bool grow = m_tile > m_ref + 8.f;          // also true for the first finite maximum
            if (__any_sync(0xffffffffu, grow) && it > 0) {
                // O is in use until the P·V of the tile before is done
                if (!ft_wait(ft_smem(p_empty), (it - 1) & 1, true)) { *failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const float f = grow ? exp2f(m_ref - m_tile) : 1.f;      // exp2(-inf) = 0: nothing was summed yet
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    float v[32];
                    ft_ld32(tmem_o + lane_addr + c, v);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= f;
                    ft_st32(tmem_o + lane_addr + c, v);
                }
                l_run *= f;
            }
            if (grow) m_ref = m_tile;
            // a row that has seen no key yet keeps m_ref = -inf; its scores are all masked (-inf) and must
            // give 0, not 2^(-inf + inf)
            const float neg_ref = m_ref > -INFINITY ? -m_ref : 0.f;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};                // partial sums by chunk, so that the adds overlap
            // P goes back into tensor memory, over the scores it came from: a 32-bit column holds two
            // neighbouring keys as bfloat16, the layout the next MMA takes its A operand in.  That buffer is
            // free: the Q·K^T that wrote these scores was issued only after the P·V that read the P before last
            // from it had completed.
            float packed[FT_BN / 2];
#pragma unroll
            for (int j = 0; j < FT_BN; j += 2) {
                const float p0 = ft_exp2(fmaf(sv[j], scale_log2, neg_ref));
                const float p1 = ft_exp2(fmaf(sv[j + 1], scale_log2, neg_ref));
                rs4[(j >> 1) & 3] += p0 + p1;
                __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                packed[j >> 1] = __uint_as_float(*reinterpret_cast<uint32_t*>(&pk));
            }
            ft_st32(s_addr, packed);
            l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            // A thread that is a whole tile ahead of the slowest must not arrive again before the phase of the
            // tile before is complete: its second arrival would stand in for the slow thread's first, and the
            // P·V would start without that thread's rows of P.  (While P went through shared memory, waiting for
            // the P·V of the tile before kept the threads together.)
            if (it > 0 && !ft_wait(ft_smem(p_full), (it - 1) & 1, true)) { *failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            ft_arrive(ft_smem(p_full));
        }
        // The last tile's P·V, then O / l.  (A barrier of its own: the softmax threads no longer follow every
        // phase of p_empty, and a wait by parity cannot tell a phase that is two behind from one that is done.)
        if (ok && !ft_wait(ft_smem(o_done), 0, true)) { *failed = 1; ok = false; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (ok) {
            const float inv = 1.f / l_run;
            bf16* orow = out + ((size_t)(tok0 + min(i_row, len - 1)) * nh + h) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                float v[32];
                ft_ld32(tmem_o + lane_addr + c, v);           // (all lanes take part in the load)
                if (i_row < len) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        __nv_bfloat162 a = __floats2bfloat162_rn(v[d] * inv, v[d + 1] * inv);
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(v[d + 2] * inv, v[d + 3] * inv);
                        __nv_bfloat162 c2 = __floats2bfloat162_rn(v[d + 4] * inv, v[d + 5] * inv);
                        __nv_bfloat162 d2 = __floats2bfloat162_rn(v[d + 6] * inv, v[d + 7] * inv);
                        *reinterpret_cast<uint4*>(orow + c + d) =
                            make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b2),
                                       *reinterpret_cast<uint32_t*>(&c2), *reinterpret_cast<uint32_t*>(&d2));
                    }
                }
            }
        }
    }
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && *failed && status) atomicOr(status, 4);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_s), "r"(256u) : "memory");
    }
}

static int ft_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

template <int HD, bool PAGED>
static int ft_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const int* block_table,
                     int table_width, int ring_pages, const int* cu_seqlens, const int* start_pos, int n_seqs,
                     int n_tokens, int window, float scale, bf16* out, int nh, int nkv, int* status,
                     cudaStream_t stream) {
    constexpr int SMEM = (HD / 64) * (FT_SUB_BYTES + 4 * FT_KV_SUB_BYTES) + 256;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(flash_prefill_tc_kernel<HD, PAGED>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const dim3 grid(nh, (n_tokens + FT_BM - 1) / FT_BM + n_seqs);
    return tq_launch_pdl(TQ_PDL_PREFILL_ATTENTION, flash_prefill_tc_kernel<HD, PAGED>, grid, dim3(FT_THREADS), SMEM, stream,
                         mq, mk, mv, block_table, table_width, ring_pages, cu_seqlens, start_pos, n_seqs, window,
                         scale * 1.4426950408889634f, out, nh, nkv, status);
}

// q, out [T, nh * hd] bfloat16.  Keys/values: packed [T, nkv * hd] (every
// sequence then starts at position 0 in this step) or pages
// [n_pages, nkv, 64, hd].  Returns cudaErrorNotSupported (801) for head sizes
// other than 64 and 128 or pages that are not 64 tokens.
TQ_API int tq_flash_prefill_tc(const void* q, const void* k_packed, const void* v_packed, const void* k_pages,
                               const void* v_pages, long long n_pages, const int* block_table, int table_width,
                               int ring_pages, int page_tokens, const int* cu_seqlens, const int* start_pos, int n_seqs,
                               int n_tokens, int window, float scale, void* out, int nh, int nkv, int hd, int* status,
                               cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (nkv <= 0 || nh % nkv || (hd != 64 && hd != 128)) return (int)cudaErrorNotSupported;
    if ((long long)(n_tokens + FT_BM - 1) / FT_BM + n_seqs > 65535) return (int)cudaErrorNotSupported;   // grid.y
    const bool paged = k_packed == nullptr;
    if (paged && (page_tokens != 64 || !k_pages || !v_pages || !block_table)) return (int)cudaErrorNotSupported;
    CUtensorMap mq, mk, mv;
    int st = ft_map(&mq, q, (uint64_t)n_tokens, (uint64_t)nh * hd, (uint64_t)nh * hd, FT_BM);
    if (st) return st;
    if (paged) {
        st = ft_map(&mk, k_pages, (uint64_t)n_pages * nkv * 64, (uint64_t)hd, (uint64_t)hd, 64);
        if (!st) st = ft_map(&mv, v_pages, (uint64_t)n_pages * nkv * 64, (uint64_t)hd, (uint64_t)hd, 64);
    } else {
        st = ft_map(&mk, k_packed, (uint64_t)n_tokens, (uint64_t)nkv * hd, (uint64_t)nkv * hd, FT_BN);
        if (!st) st = ft_map(&mv, v_packed, (uint64_t)n_tokens, (uint64_t)nkv * hd, (uint64_t)nkv * hd, FT_BN);
    }
    if (st) return st;
#define TQ_FT(H, P) return ft_launch<H, P>(mq, mk, mv, block_table, table_width, ring_pages, cu_seqlens, start_pos, \
                                           n_seqs, n_tokens, window, scale, (bf16*)out, nh, nkv, status, stream)
    if (hd == 128 && paged) TQ_FT(128, true);
    if (hd == 128 && !paged) TQ_FT(128, false);
    if (hd == 64 && paged) TQ_FT(64, true);
    TQ_FT(64, false);
#undef TQ_FT
}
