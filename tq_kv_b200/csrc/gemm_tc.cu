// Matrix product on the 5th-generation tensor cores of sm_100a:
//   C[M,N] = A[M,K] · B[N,K]^T     (bfloat16 operands, float32 accumulation)
// with tcgen05.mma issued by one thread, operands brought into shared memory
// by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a 4-stage mbarrier
// pipeline, the accumulator in tensor memory (TMEM) and read back with
// tcgen05.ld for the epilogue.  Tiles are 128 x 256; one persistent block per
// SM walks its share of them.
//
// Epilogues (fused, float32): plain store (float32 or bfloat16, optional
// bias), accumulate into a float32 C (the residual sum,
// src/models/turbo_generic.rs:1969,1980), and SwiGLU gating
// (src/models/turbo_generic.rs:105-110): B then holds the gate rows followed
// by the up rows, a tile's 256 accumulator columns are 128 gate columns and
// the 128 up columns of the same outputs, and silu(gate) * up is written.
//
// Roles: warp 0 lane 0 issues TMA loads, warp 1 lane 0 issues the MMAs
// (warp 1 also allocates and frees TMEM), warps 2..5 run the epilogue of one
// accumulator while the MMAs fill the other: warp w reads TMEM lanes
// 32 (w % 4) .. +31, lays [32 x 32] pieces into shared memory and hands them
// to TMA, as a store or, for the residual sum, as a reduce-add done in the L2.
// Every wait on an mbarrier is bounded: when a bound is hit the role raises
// a flag, stops, the others run into their own bounds, the block still frees
// its TMEM, raises a bit in *status and returns: an error, not a hang.
//
// When the tiles do not fill the last round of the persistent blocks (224
// tiles on 148 SMs), or are fewer than the SMs, the float32 products cut
// those tiles along K into 2 to 8 shares; the shares meet in C through the
// reduce-add, so for those tiles the order of the float additions is not
// fixed.
//
// From 129 rows on the same product runs on pairs of SMs (gemm_tc_pair_kernel
// below): tcgen05.mma with cta_group::2 on 256 x 256 tiles, each block of a
// 2-block cluster holding half of A's rows and half of the B tile, which cuts
// what an SM loads per step from 48 to 32 KB (measured: 5 % off the prefill).
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BN 256
#define TC_BK 64
#define TC_STAGES 4
#define TC_THREADS 192
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_B_BYTES (TC_BN * TC_BK * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_EPI_BYTES (32 * 32 * 4)        /* a warp's [32 rows x 32 columns] float32 piece on its way out */
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 4 * 2 * TC_EPI_BYTES + 256)
#define TC_WAIT_CYCLES (4000000000ll)     /* about two seconds of SM clock */

#define EPI_STORE 0
#define EPI_ACCUM 1
#define EPI_SWIGLU 2

// ---- PTX wrappers -------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: false if the phase did not complete within about two seconds.
// `backoff`: sleep between polls (for the many threads that only wait for the accumulator).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, bool backoff = false) {
    const long long t0 = clock64();
    for (uint32_t i = 1;; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (backoff) __nanosleep(200);
        if ((i & 255u) == 0 && clock64() - t0 > TC_WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 columns of 32-bit TMEM cells -> 32 registers per thread (thread i = lane i of the warp's quarter)
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle:
// rows are 128 bytes, groups of 8 rows (1024 bytes) follow each other.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);            // start address
    d |= (uint64_t)0 << 16;                            // leading byte offset (unused: one swizzle atom along K)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // layout: 128-byte swizzle
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M x N.
__device__ __forceinline__ uint32_t instr_desc(uint32_t m, uint32_t n) {
    return (1u << 4)            // D format f32
         | (1u << 7)            // A format bf16
         | (1u << 10)           // B format bf16
         | ((n >> 3) << 17)     // N / 8
         | ((m >> 4) << 24);    // M / 16
}

// ---- the epilogue of one accumulator, one warp's 32 rows --------------------------------
// A thread holds 32 neighbouring columns of its row; the warp lays its [32 x 32] piece into shared memory
// (rows of 128 bytes, 16-byte chunks swizzled so that the 32 rows do not meet in a bank) and one lane hands
// it to TMA: a store, or for the residual sum a reduce-add, which adds in the L2 without reading C into the
// SM and is the same operation for whole tiles and for shares of K.  TMA clips rows >= M and columns >= N.
// Two buffers per warp (st): a piece is written while the one before is on its way; `piece` counts them.
template <int EPI, typename TO>
__device__ __forceinline__ void tc_epilogue_item(uint32_t t_row, unsigned char* st, uint32_t& piece,
                                                 const CUtensorMap* map_c_ptr, const float* __restrict__ bias, int n0,
                                                 int row0, int M, int N, int part, int lane) {
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const bool rows_live = row0 < M;                  // a warp whose rows all lie past M stores nothing
#pragma unroll 1
    for (int c = 0; c < OUT_COLS; c += 32) {
        if (n0 + c >= N) break;
        float v[32];
        if (EPI == EPI_SWIGLU) {
            float u[32];
            tc_ld32(t_row + c, v);
            tc_ld32(t_row + TC_BN / 2 + c, u);
            tc_wait_ld();
            // silu(g) * u.  A bfloat16 result keeps 8 bits: the fast exponential and division (2 ulp of float32)
            // cost a third of the exact ones' instructions, which a short K cannot hide under its MMAs.
#pragma unroll
            for (int j = 0; j < 32; ++j)
                v[j] = sizeof(TO) == 2 ? __fdividef(v[j], 1.f + __expf(-v[j])) * u[j]
                                       : (v[j] / (1.f + expf(-v[j]))) * u[j];
        } else {
            tc_ld32(t_row + c, v);
            tc_wait_ld();
        }
        if (bias != nullptr && part <= 0) {           // one share of a tile adds the bias
            const int col = n0 + c + lane;
            const float mine = col < N ? bias[col] : 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, mine, j);
        }
        if (!rows_live) continue;
        unsigned char* pb = st + (piece & 1) * TC_EPI_BYTES;
        // the piece before last used this buffer: its bytes must have been read
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");
        __syncwarp();
        if (sizeof(TO) == 4) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(pb + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                    make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 a = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                __nv_bfloat162 c2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                __nv_bfloat162 d2 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                *reinterpret_cast<uint4*>(pb + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) =
                    make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b2),
                               *reinterpret_cast<uint32_t*>(&c2), *reinterpret_cast<uint32_t*>(&d2));
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            if (EPI == EPI_ACCUM)
                asm volatile(
                    "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                    ::"l"(map_c_ptr), "r"(n0 + c), "r"(row0), "r"(smem_u32(pb)) : "memory");
            else
                asm volatile(
                    "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                    ::"l"(map_c_ptr), "r"(n0 + c), "r"(row0), "r"(smem_u32(pb)) : "memory");
            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        }
        ++piece;
    }
}

// ---- the kernel -------------------------------------------------------------------
// Persistent: one block per SM walks the output tiles t = blockIdx.x, + gridDim.x, ...
// (tiles that share a B tile are neighbours, so they meet in L2).  Two
// accumulators of 256 TMEM columns alternate, so the MMAs of a tile overlap
// the epilogue of the tile before.  b_rows_second: SwiGLU only — row offset
// of the up rows in B (the number of outputs).
template <int EPI, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const float* __restrict__ bias, int M, int N, int K,
               int b_rows_second, int n_whole, int parts, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + TC_STAGES * TC_STAGE_BYTES;       // [4 warps][2 buffers][32 rows][128 bytes]
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 4 * 2 * TC_EPI_BYTES);
    // bars: full[S], empty[S], acc_full[2], acc_empty[2]; then the TMEM address and a failure flag
    uint64_t* full = bars;
    uint64_t* empty = bars + TC_STAGES;
    uint64_t* acc_full = bars + 2 * TC_STAGES;
    uint64_t* acc_empty = bars + 2 * TC_STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 4);
    volatile uint32_t* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // output columns of a tile; with SwiGLU a tile yields 128 outputs from 128 gate + 128 up rows of B
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const int tiles_m = (M + TC_BM - 1) / TC_BM;
    const int tiles_n = (N + OUT_COLS - 1) / OUT_COLS;
    const int n_tiles = tiles_m * tiles_n;
    const int k_all = (K + TC_BK - 1) / TC_BK;
    // Work items: the first n_whole tiles whole; the others (a short last round, residual epilogue only) cut
    // into `parts` shares of K each, so that the last round keeps every SM busy.  Item w -> (tile, k range).
    const int n_items = n_whole + (n_tiles - n_whole) * parts;
    const int k_share = (k_all + parts - 1) / parts;
    auto item = [&](int w, int& t, int& k_lo, int& k_cnt, int& part) {
        if (w < n_whole) { t = w; k_lo = 0; k_cnt = k_all; part = -1; return; }
        const int r = w - n_whole;
        t = n_whole + r / parts;
        part = r % parts;
        k_lo = min(k_all, part * k_share);
        k_cnt = min(k_all, k_lo + k_share) - k_lo;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);          // one arrival per epilogue warp
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * TC_BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch (common.cuh): barriers and tensor memory are set up under the tail of the
    // kernel before; its results (A, and C where the product adds to it) are touched only from here on.
    pdl_wait();
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: TMA loads ----
            uint32_t it = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
                int t, k_lo, k_iters, part;
                item(w, t, k_lo, k_iters, part);
                const int m0 = (t % tiles_m) * TC_BM, n0 = (t / tiles_m) * OUT_COLS;
                for (int i = 0; i < k_iters; ++i, ++it) {
                    const int s = it % TC_STAGES;
                    if (!mbar_wait(smem_u32(&empty[s]), ((it / TC_STAGES) & 1) ^ 1)) { *failed = 1; ok = false; break; }
                    const uint32_t fb = smem_u32(&full[s]);
                    const uint32_t a_dst = smem_u32(tiles + s * TC_STAGE_BYTES);
                    const uint32_t b_dst = a_dst + TC_A_BYTES;
                    mbar_expect_tx(fb, TC_STAGE_BYTES);
                    const int kc = (k_lo + i) * TC_BK;
                    tma_load_2d(a_dst, &map_a, kc, m0, fb);
                    if (EPI == EPI_SWIGLU) {
                        tma_load_2d(b_dst, &map_b, kc, n0, fb);                                  // gate rows
                        tma_load_2d(b_dst + TC_B_BYTES / 2, &map_b, kc, b_rows_second + n0, fb); // up rows
                    } else {
                        tma_load_2d(b_dst, &map_b, kc, n0, fb);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----
            const uint32_t idesc = instr_desc(TC_BM, TC_BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++local) {
                int t, k_lo, k_iters, part;
                item(w, t, k_lo, k_iters, part);
                const uint32_t buf = local & 1;
                if (!mbar_wait(smem_u32(&acc_empty[buf]), ((local >> 1) & 1) ^ 1)) { *failed = 1; ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int i = 0; i < k_iters; ++i, ++it) {
                    const int s = it % TC_STAGES;
                    if (!mbar_wait(smem_u32(&full[s]), (it / TC_STAGES) & 1)) { *failed = 1; ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * TC_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TC_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        // 16 elements of K = 32 bytes further inside the swizzle atom
                        tc_mma(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                               (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&empty[s]));             // frees the stage when these MMAs are done
                }
                if (ok) tc_commit(smem_u32(&acc_full[buf]));    // this tile's accumulator is complete
            }
        }
    } else {
        // ---- epilogue warps: warp w reads TMEM lanes 32 * (w % 4) .. + 31 = rows of the tile.  A thread holds
        // 32 neighbouring columns of its row; the warp lays its [32 x 32] piece into shared memory (rows of 128
        // bytes, 16-byte chunks swizzled so that the 32 rows do not meet in a bank) and one lane hands it to
        // TMA: a store, or for the residual sum a reduce-add, which adds in the L2 without reading C into the
        // SM and is the same operation for whole tiles and for shares of K.  TMA clips rows >= M and columns
        // >= N.  Two buffers per warp: a piece is written while the one before is on its way. ----
        const int quarter = warp & 3;
        unsigned char* st = staging + (warp - 2) * 2 * TC_EPI_BYTES;
        uint32_t local = 0, piece = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++local) {
            int t, k_lo, k_iters, part;
            item(w, t, k_lo, k_iters, part);
            const int m0 = (t % tiles_m) * TC_BM, n0 = (t / tiles_m) * OUT_COLS;
            const uint32_t buf = local & 1;
            if (!mbar_wait(smem_u32(&acc_full[buf]), (local >> 1) & 1, true)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TC_BN;
            const int row0 = m0 + quarter * 32;
            tc_epilogue_item<EPI, TO>(t_row, st, piece, &map_c, bias, n0, row0, M, N, part, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");   // all pieces have landed
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *failed && status) atomicOr(status, 2);   // a wait ran out: the result is not valid
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)(2 * TC_BN))
                     : "memory");
    }
}

// ---- the same product on pairs of SMs (tcgen05 cta_group::2) ------------------------------
// A cluster of two blocks owns a 256 x 256 tile: block r of the pair holds rows 128 r .. of A and rows
// 128 r .. of the B tile (with SwiGLU: block 0 the gate rows, block 1 the up rows), and one thread of
// block 0 issues MMAs of M = 256 that read both blocks' shared memory and write each block's half of the
// accumulator into its own TMEM.  Per 64 of K a block loads 32 KB instead of 48, which is what the L2 has
// to deliver to an SM; the stages saved go into a deeper pipeline (6).
//   full[s]       block 0's: its producer announces both blocks' bytes, both blocks' TMA loads report there
//   empty[s]      each block's own, freed by the MMAs' commit, which is multicast to both blocks
//   acc_full[b]   each block's own, by commit multicast
//   acc_empty[b]  block 0's: the epilogue warps of both blocks arrive there (2 x 4)
// Every wait is bounded as above; whatever happens, both blocks reach the cluster barrier at the end, so
// that neither leaves while the other may still touch its shared memory or barriers.
#define T2_STAGES 6
#define T2_STAGE_BYTES (2 * TC_A_BYTES)   /* A: 128 x 64, B: this block's 128 x 64 */
#define T2_SMEM_BYTES (T2_STAGES * T2_STAGE_BYTES + 1024 + 4 * 2 * TC_EPI_BYTES + 256)

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the address of a shared-memory location of block `rank` of the cluster, in the cluster's window
__device__ __forceinline__ uint32_t cluster_map(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {     // arrives on `bar` in both blocks of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int EPI, typename TO>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const float* __restrict__ bias, int M, int N, int K,
                    int b_rows_second, int n_whole, int parts, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = tiles + T2_STAGES * T2_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 4 * 2 * TC_EPI_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + T2_STAGES;
    uint64_t* acc_full = bars + 2 * T2_STAGES;
    uint64_t* acc_empty = bars + 2 * T2_STAGES + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T2_STAGES + 4);
    volatile uint32_t* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                  // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const int tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    const int tiles_n = (N + OUT_COLS - 1) / OUT_COLS;
    const int n_tiles = tiles_m * tiles_n;
    const int k_all = (K + TC_BK - 1) / TC_BK;
    const int n_items = n_whole + (n_tiles - n_whole) * parts;
    const int k_share = (k_all + parts - 1) / parts;
    auto item = [&](int w, int& t, int& k_lo, int& k_cnt, int& part) {
        if (w < n_whole) { t = w; k_lo = 0; k_cnt = k_all; part = -1; return; }
        const int r = w - n_whole;
        t = n_whole + r / parts;
        part = r % parts;
        k_lo = min(k_all, part * k_share);
        k_cnt = min(k_all, k_lo + k_share) - k_lo;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < T2_STAGES; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 8);          // one arrival per epilogue warp of either block
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {                                       // the same warp of both blocks: one allocation for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * TC_BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // the peer's barriers exist from here on
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                                            // (as in the single-SM form)
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both blocks): this block's A rows and its half of the B tile ----
            uint32_t it = 0;
            bool ok = true;
            for (int w = pair; w < n_items && ok; w += n_pairs) {
                int t, k_lo, k_iters, part;
                item(w, t, k_lo, k_iters, part);
                const int m0 = (t % tiles_m) * 2 * TC_BM + (int)rank * TC_BM;
                const int n0 = (t / tiles_m) * OUT_COLS;
                const int b_row = EPI == EPI_SWIGLU ? (rank == 0 ? n0 : b_rows_second + n0) : n0 + (int)rank * (TC_BN / 2);
                for (int i = 0; i < k_iters; ++i, ++it) {
                    const int s = it % T2_STAGES;
                    if (!mbar_wait(smem_u32(&empty[s]), ((it / T2_STAGES) & 1) ^ 1)) { *failed = 1; ok = false; break; }
                    const uint32_t fb = cluster_map(smem_u32(&full[s]), 0);
                    if (rank == 0) mbar_expect_tx(smem_u32(&full[s]), 2 * T2_STAGE_BYTES);
                    const uint32_t a_dst = smem_u32(tiles + s * T2_STAGE_BYTES);
                    const int kc = (k_lo + i) * TC_BK;
                    tma_load_2d_pair(a_dst, &map_a, kc, m0, fb);
                    tma_load_2d_pair(a_dst + TC_A_BYTES, &map_b, kc, b_row, fb);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (block 0 only): D[256 x 256] over both blocks ----
            const uint32_t idesc = instr_desc(2 * TC_BM, TC_BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int w = pair; w < n_items && ok; w += n_pairs, ++local) {
                int t, k_lo, k_iters, part;
                item(w, t, k_lo, k_iters, part);
                const uint32_t buf = local & 1;
                if (!mbar_wait(smem_u32(&acc_empty[buf]), ((local >> 1) & 1) ^ 1)) { *failed = 1; ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int i = 0; i < k_iters; ++i, ++it) {
                    const int s = it % T2_STAGES;
                    if (!mbar_wait(smem_u32(&full[s]), (it / T2_STAGES) & 1)) { *failed = 1; ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + s * T2_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TC_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        tc_mma_pair(d_tmem, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                                    (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(smem_u32(&empty[s]));        // frees the stage in both blocks
                }
                if (ok) tc_commit_pair(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---- epilogue warps (both blocks): this block's 128 rows of the tile ----
        const int quarter = warp & 3;
        unsigned char* st = staging + (warp - 2) * 2 * TC_EPI_BYTES;
        uint32_t local = 0, piece = 0;
        bool ok = true;
        for (int w = pair; w < n_items && ok; w += n_pairs, ++local) {
            int t, k_lo, k_iters, part;
            item(w, t, k_lo, k_iters, part);
            const int m0 = (t % tiles_m) * 2 * TC_BM + (int)rank * TC_BM, n0 = (t / tiles_m) * OUT_COLS;
            const uint32_t buf = local & 1;
            if (!mbar_wait(smem_u32(&acc_full[buf]), (local >> 1) & 1, true)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TC_BN;
            tc_epilogue_item<EPI, TO>(t_row, st, piece, &map_c, bias, n0, m0 + quarter * 32, M, N, part, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n"
                             ::"r"(cluster_map(smem_u32(&acc_empty[buf]), 0)) : "memory");
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // nobody leaves while its peer may still need it
    if (threadIdx.x == 0 && *failed && status) atomicOr(status, 2);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)(2 * TC_BN))
                     : "memory");
    }
}

// ---- host side ------------------------------------------------------------------
// rows x cols bfloat16, row stride ld elements; box = box_rows x 64 columns, 128-byte swizzle
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {TC_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// C: rows x cols of float32 or bfloat16, row stride ld elements; box = 32 rows x 32 columns, swizzled over the
// row's bytes (128 or 64) as the epilogue lays it out
static int make_map_c(CUtensorMap* map, const void* base, bool f32, uint64_t rows, uint64_t cols, uint64_t ld) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * (f32 ? 4 : 2)};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = cuTensorMapEncodeTiled(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                        const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// Into how many shares of K the tiles of the last, incomplete round are cut: rem * parts pieces of 1 / parts of
// a tile each take ceil(rem * parts / sms) / parts tile times, plus a little for each share's epilogue.
// *gain (optional): that time over the uncut round's.
static int tc_last_round_parts(int n_tiles, int sms, int K, double* gain) {
    const int rem = n_tiles % sms, k_all = (K + TC_BK - 1) / TC_BK;
    int parts = 1;
    double best = 1.0;
    if (rem > 0 && !tq_deterministic()) {
        for (int p = 2; p <= 8 && k_all / p >= 8; ++p) {
            const double t = (double)((rem * p + sms - 1) / sms) / p + 0.02 * p;
            if (t < best - 1e-9) { best = t; parts = p; }
        }
    }
    if (gain) *gain = best;
    return parts;
}

static int tc_sm_count() { return tq_sm_count(); }

template <int EPI, typename TO>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const float* bias, int M, int N,
                     int K, int b_rows_second, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             TC_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const int n_tiles = ((N + OUT_COLS - 1) / OUT_COLS) * ((M + TC_BM - 1) / TC_BM);
    const int sm_count = tc_sm_count();
    // The tiles of an incomplete last round (all tiles, if they are fewer than the SMs) are cut along K into
    // `parts` shares (residual epilogue only: the shares add up in C), with the number of shares that lets
    // the round end soonest.
    int n_whole = n_tiles, parts = 1;
    if (EPI == EPI_ACCUM) parts = tc_last_round_parts(n_tiles, sm_count, K, nullptr);
    if (parts > 1) n_whole = n_tiles - n_tiles % sm_count;
    const int n_items = n_whole + (n_tiles - n_whole) * parts;
    const int grid = n_items < sm_count ? n_items : sm_count;
    return tq_launch_pdl(TQ_PDL_GEMM_TC, gemm_tc_kernel<EPI, TO>, dim3(grid), dim3(TC_THREADS), TC_SMEM_BYTES, stream, ma, mb,
                         mc, bias, M, N, K, b_rows_second, n_whole, parts, status);
}

// The pair form: 256-row tiles on clusters of two blocks.
template <int EPI, typename TO>
static int launch_tc_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const float* bias, int M,
                          int N, int K, int b_rows_second, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             T2_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const int n_tiles = ((N + OUT_COLS - 1) / OUT_COLS) * ((M + 2 * TC_BM - 1) / (2 * TC_BM));
    const int pairs = tc_sm_count() / 2 > 0 ? tc_sm_count() / 2 : 1;
    int n_whole = n_tiles, parts = 1;
    if (EPI == EPI_ACCUM) parts = tc_last_round_parts(n_tiles, pairs, K, nullptr);
    if (parts > 1) n_whole = n_tiles - n_tiles % pairs;
    const int n_items = n_whole + (n_tiles - n_whole) * parts;
    const int grid = 2 * (n_items < pairs ? n_items : pairs);
    return tq_launch_pdl(TQ_PDL_GEMM_TC, gemm_tc_pair_kernel<EPI, TO>, dim3(grid), dim3(TC_THREADS), T2_SMEM_BYTES, stream,
                         ma, mb, mc, bias, M, N, K, b_rows_second, n_whole, parts, status);
}

// 0: pairs of SMs for products of more than 128 rows, single SMs otherwise; 1: single SMs always; 2: pairs always.
// Starts from the environment variable TQ_GEMM_TC_MODE (a tuning aid), else 0.
static int g_tc_mode = -1;
TQ_API void tq_gemm_tc_mode(int mode) { g_tc_mode = mode; }
static int tc_mode() {
    if (g_tc_mode < 0) {
        const char* e = getenv("TQ_GEMM_TC_MODE");
        g_tc_mode = e ? atoi(e) : 0;
        if (g_tc_mode < 0 || g_tc_mode > 2) g_tc_mode = 0;
    }
    return g_tc_mode;
}

// A [M, K] and B [N, K] (or [2N, K] with epilogue 2) bfloat16 with row strides
// lda / ldb (elements, multiples of 8; bases 16-byte aligned); C [M, N] with
// row stride ldc (base and row stride in bytes multiples of 16), float32 or
// bfloat16 (epilogue 1 needs float32).
// status: device int, bit 1 is raised if a pipeline wait ran out.
TQ_API int tq_gemm_tc(const void* A, const void* B, const float* bias, void* C, int c_dtype, int M, int N, int K,
                      int lda, int ldb, int ldc, int epilogue, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7)) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_ACCUM && c_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    if (c_dtype != TQ_F32 && c_dtype != TQ_BF16) return (int)cudaErrorInvalidValue;
    // C leaves through TMA: 16-byte aligned base and row stride
    if ((reinterpret_cast<uintptr_t>(C) & 15) || ((size_t)ldc * (c_dtype == TQ_F32 ? 4 : 2)) % 16)
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    int st = make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM);
    if (st) return st;
    const bool pair = tc_mode() == 2 || (tc_mode() == 0 && M > TC_BM);
    const uint64_t b_rows = epilogue == EPI_SWIGLU ? 2ull * N : (uint64_t)N;
    // a block loads 128 rows of B at a time in the pair form and with SwiGLU, else the tile's 256
    st = make_map(&mb, B, b_rows, (uint64_t)K, (uint64_t)ldb, (pair || epilogue == EPI_SWIGLU) ? TC_BN / 2 : TC_BN);
    if (st) return st;
    CUtensorMap mc;
    st = make_map_c(&mc, C, c_dtype == TQ_F32, (uint64_t)M, (uint64_t)N, (uint64_t)ldc);
    if (st) return st;
#define TQ_TC(E, T)                                                                                   \
    return pair ? launch_tc_pair<E, T>(ma, mb, mc, bias, M, N, K, N, status, stream)                  \
                : launch_tc<E, T>(ma, mb, mc, bias, M, N, K, N, status, stream)
    if (epilogue == EPI_STORE && c_dtype == TQ_F32) {
        // A float32 result whose tiles fill the last round badly (few rows: 72 tiles on 148 SMs) is cleared and
        // then summed from shares of K like the residual product; worth it when the last round is most of the
        // work and the shares cut it by a third or more.
        const int n_tiles = ((N + TC_BN - 1) / TC_BN) * ((M + (pair ? 2 : 1) * TC_BM - 1) / ((pair ? 2 : 1) * TC_BM));
        double gain = 1.0;
        const int sms = pair ? tc_sm_count() / 2 : tc_sm_count();
        if (n_tiles < 2 * sms && tc_last_round_parts(n_tiles, sms, K, &gain) > 1 && gain <= 0.67) {
            cudaError_t e = cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, stream);
            if (e != cudaSuccess) return (int)e;
            TQ_TC(EPI_ACCUM, float);
        }
        TQ_TC(EPI_STORE, float);
    }
    if (epilogue == EPI_STORE && c_dtype == TQ_BF16) TQ_TC(EPI_STORE, bf16);
    if (epilogue == EPI_ACCUM) TQ_TC(EPI_ACCUM, float);
    if (epilogue == EPI_SWIGLU && c_dtype == TQ_F32) TQ_TC(EPI_SWIGLU, float);
    if (epilogue == EPI_SWIGLU && c_dtype == TQ_BF16) TQ_TC(EPI_SWIGLU, bf16);
#undef TQ_TC
    return (int)cudaErrorInvalidValue;
}
