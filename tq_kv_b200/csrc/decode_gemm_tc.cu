// Weight-streaming product for decoding batches of up to 64 rows on the
// tcgen05 tensor cores, operands swapped: the 128 rows of a W tile are the
// "M" side of the instruction, the (padded) batch is its "N" side, so the
// accumulator D[128 weight rows x batch] sits in TMEM with one weight row per
// lane.  Y[M,N] = X[M,K] · W[N,K]^T.
//
// A block owns 128 output columns (64 with SwiGLU: 64 gate rows and the 64 up
// rows of the same outputs share a tile) and a share of K; W and X tiles come
// in by TMA through a 4-stage mbarrier pipeline (16 KB of W per stage; two
// blocks fit an SM, so ~128 KB of weights are in flight per SM and one
// block's epilogue runs under the other's loads).  Where 128-row tiles alone give
// too few blocks to pull the HBM bandwidth, a thread-block cluster of 2, 4 or
// 8 blocks splits K; the blocks then share out the tile's outputs and each
// adds the partial sums of its share, read from all blocks' shared memory in
// rank order (no atomics: the result does not depend on scheduling).  Epilogues as in skinny_gemm.cu: bias, SwiGLU
// gating, adding into the float32 residual stream, float32 or bfloat16 out.
//
// Float32 results without gating have a second way to split K (REDUCE): the
// shares are independent blocks, as many as fill the GPU's block slots (two an SM) once, and each hands
// its partial tile to TMA as a reduce-add, which sums in the L2
// (cp.reduce.async.bulk.tensor); a result that is not added to the residual
// stream is cleared first.  No cluster, no exchange through shared memory;
// the order of the float additions of one output is then not fixed.
//
// All waits on mbarriers are bounded (see gemm_tc.cu): a wait that runs out
// raises a bit in *status, the block still frees its TMEM and returns.
#include <cooperative_groups.h>
#include <cuda.h>

#include "common.cuh"
namespace cg = cooperative_groups;

#define DG_ROWS 128                 // weight rows per tile (TMEM lanes)
#define DG_BK 64
#define DG_THREADS 192
#define DG_W_BYTES (DG_ROWS * DG_BK * 2)
#define DG_WAIT_CYCLES (4000000000ll)

__device__ __forceinline__ uint32_t dg_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool dg_wait(uint32_t bar, uint32_t parity, bool backoff = false) {
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
        if ((i & 255u) == 0 && clock64() - t0 > DG_WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void dg_tma(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t dg_desc(uint32_t saddr) {      // K-major tile, 128-byte swizzle (see gemm_tc.cu)
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void dg_ld32(uint32_t taddr, float* v) {
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

// MP: padded batch (32 or 64) = columns of the accumulator.
// DG_STAGES: 4 (96 KB per block: two blocks fit an SM, one's epilogue runs under the other's loads).  Inside the
// decode step five stages were slower (200 KB an SM leave the next kernel no room to set itself up), eight too.
//
// NORM (cluster form, up to 16 batch rows): the activations are the float32 residual stream H [M, K] and the
// weights G [K] of an RMS norm (src/models/turbo_generic.rs:41-51) instead of bfloat16 rows.  The four warps
// that later run the epilogue build each stage's X tile themselves: every thread fetches eight values of one
// row through a small cp.async ring of its own (four stages ahead of the tile it writes), multiplies them with
// g, rounds to bfloat16 and stores them where the 128-byte swizzle of the tile wants them; the squares are
// summed on the way, each block over its share of K, and the shares meet with the partial products in the
// cluster's exchange, where every output is scaled by 1 / sqrt(mean(h^2) + eps) of its batch row.  So the norm
// needs no kernel and no trip through memory of its own.
#define DG_NORM_ROWS 16
#define DG_HRING 4
template <int MP, bool SWIGLU, typename TO, int DG_STAGES, bool REDUCE, bool NORM = false>
__global__ void __launch_bounds__(DG_THREADS, 2)
decode_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      const __grid_constant__ CUtensorMap map_y, const float* __restrict__ bias, TO* __restrict__ Y,
                      int M, int N, int K, int ldy, int accumulate, int k_splits, int* __restrict__ status,
                      const float* __restrict__ H = nullptr, int ldh = 0, const float* __restrict__ G = nullptr,
                      float eps = 0.f) {
    static_assert(!NORM || (!REDUCE && MP == 32), "the folded norm runs in the cluster form with up to 16 rows");
    constexpr int X_BYTES = MP * DG_BK * 2;
    constexpr int STAGE_BYTES = DG_W_BYTES + X_BYTES;
    constexpr int OUT_COLS = SWIGLU ? DG_ROWS / 2 : DG_ROWS;
    constexpr int RED_LD = MP + 1;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // the partial sums reuse the first stages once the pipeline has drained: [128 weight rows][MP + 1]
    float* red = reinterpret_cast<float*>(tiles);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + DG_STAGES * STAGE_BYTES);
    uint64_t* full = bars;
    uint64_t* empty = bars + DG_STAGES;
    uint64_t* acc_full = bars + 2 * DG_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * DG_STAGES + 1);
    volatile uint32_t* failed = tmem_slot + 1;
    float* ss_part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(bars) + 128);   // NORM: [16] sums of squares
    unsigned char* hring = reinterpret_cast<unsigned char*>(bars) + 256;                       // NORM: [DG_HRING][128][32 B]

    cg::cluster_group cluster = cg::this_cluster();
    // shares of K: the blocks of a cluster, or (REDUCE) k_splits independent blocks in a row of the grid
    const int n_ranks = REDUCE ? k_splits : (int)cluster.num_blocks();
    const int rank = REDUCE ? (int)(blockIdx.x % k_splits) : (int)cluster.block_rank();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x / n_ranks) * OUT_COLS;
    const int k_total = (K + DG_BK - 1) / DG_BK;
    const int k_per = (k_total + n_ranks - 1) / n_ranks;
    const int k_lo = min(k_total, rank * k_per), k_hi = min(k_total, k_lo + k_per);
    const int k_iters = k_hi - k_lo;

    if (threadIdx.x == 0) {
        for (int s = 0; s < DG_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(dg_smem(&full[s])), "r"(NORM ? 2u : 1u));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(dg_smem(&empty[s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(dg_smem(acc_full)));
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(dg_smem(tmem_slot)), "r"((uint32_t)MP) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // Programmatic dependent launch (common.cuh): the weights do not depend on the kernel before, so the first
    // stages' W tiles are requested before waiting for it; X, bias and Y are touched only after pdl_wait().
    if (!(warp == 0 && lane == 0)) { pdl_wait(); pdl_launch(); }
    if (warp == 0 && lane == 0) {
        // ---- producer ----
        auto load_w = [&](int i) {
            const int s = i % DG_STAGES;
            const uint32_t fb = dg_smem(&full[s]);
            const uint32_t w_dst = dg_smem(tiles + s * STAGE_BYTES);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
                         ::"r"(fb), "r"((uint32_t)(NORM ? DG_W_BYTES : STAGE_BYTES)) : "memory");
            const int kc = (k_lo + i) * DG_BK;
            if (SWIGLU) {
                dg_tma(w_dst, &map_w, kc, n0, fb);                          // 64 gate rows
                dg_tma(w_dst + DG_W_BYTES / 2, &map_w, kc, N + n0, fb);     // the 64 up rows of the same outputs
            } else {
                dg_tma(w_dst, &map_w, kc, n0, fb);
            }
        };
        auto load_x = [&](int i) {
            const int s = i % DG_STAGES;
            dg_tma(dg_smem(tiles + s * STAGE_BYTES) + DG_W_BYTES, &map_x, (k_lo + i) * DG_BK, 0, dg_smem(&full[s]));
        };
        const int ahead = k_iters < DG_STAGES ? k_iters : DG_STAGES;     // the stages are empty at the start
        for (int i = 0; i < ahead; ++i) load_w(i);
        pdl_wait();
        pdl_launch();
        if (!NORM)
            for (int i = 0; i < ahead; ++i) load_x(i);
        for (int i = ahead; i < k_iters; ++i) {
            const int s = i % DG_STAGES;
            if (!dg_wait(dg_smem(&empty[s]), ((i / DG_STAGES) & 1) ^ 1)) { *failed = 1; break; }
            load_w(i);
            if (!NORM) load_x(i);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D[128 x MP] (+)= W_tile[128 x 64] · X_tile[MP x 64]^T ----
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MP >> 3) << 17) | ((uint32_t)(DG_ROWS >> 4) << 24);
        for (int i = 0; i < k_iters; ++i) {
            const int s = i % DG_STAGES;
            if (!dg_wait(dg_smem(&full[s]), (i / DG_STAGES) & 1)) { *failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t w_addr = dg_smem(tiles + s * STAGE_BYTES);
            const uint32_t x_addr = w_addr + DG_W_BYTES;
#pragma unroll
            for (int k = 0; k < DG_BK / 16; ++k) {
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                    ::"r"(tmem_base), "l"(dg_desc(w_addr + k * 32)), "l"(dg_desc(x_addr + k * 32)), "r"(idesc), "r"(acc)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                         ::"r"(dg_smem(&empty[s])) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                     ::"r"(dg_smem(acc_full)) : "memory");
    }
    if (NORM && warp >= 2) {
        // ---- the X tiles from the residual stream (see NORM above); these threads have passed pdl_wait() ----
        const int t = threadIdx.x - 64;                    // 0..127: row t / 8 of the tile, 16-byte piece t % 8
        const int row = t >> 3, piece = t & 7;
        const bool row_on = row < M;
        const uint4 zero = make_uint4(0, 0, 0, 0);
        for (int s = 0; s < DG_STAGES; ++s)                // rows from M on stay zero in every stage
            for (int e = t; e < X_BYTES / 16; e += 128)
                *reinterpret_cast<uint4*>(tiles + s * STAGE_BYTES + DG_W_BYTES + e * 16) = zero;
        const float* hrow = H + (size_t)(row_on ? row : 0) * ldh;
        unsigned char* mine = hring + t * 32;
        auto fetch = [&](int i) {                          // one group per turn, empty or not
            const int k = (k_lo + i) * DG_BK + piece * 8;
            if (row_on && i < k_iters && k < K) {
                const uint32_t dst = dg_smem(mine + (i % DG_HRING) * (128 * 32));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(hrow + k) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + 16), "l"(hrow + k + 4) : "memory");
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };
#pragma unroll
        for (int i = 0; i < DG_HRING - 1; ++i) fetch(i);
        float ss = 0.f;
        // the norm's weights for the next DG_HRING tiles wait in registers: they do not depend on the kernel
        // before and are asked for that many turns ahead of their use
        float4 gq[DG_HRING][2];
        auto fetch_g = [&](int i, float4* dst) {
            const int k = (k_lo + i) * DG_BK + piece * 8;
            if (i < k_iters && k < K) {
                dst[0] = *reinterpret_cast<const float4*>(G + k);
                dst[1] = *reinterpret_cast<const float4*>(G + k + 4);
            } else {
                dst[0] = dst[1] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
#pragma unroll
        for (int j = 0; j < DG_HRING; ++j) fetch_g(j, gq[j]);
        bool stop = false;
        for (int i0 = 0; i0 < k_iters && !stop; i0 += DG_HRING) {
#pragma unroll
            for (int j = 0; j < DG_HRING; ++j) {
                const int i = i0 + j;
                if (i >= k_iters || stop) break;
                const int s = i % DG_STAGES;
                const int k = (k_lo + i) * DG_BK + piece * 8;
                const bool on = row_on && k < K;
                const float4 g0 = gq[j][0], g1 = gq[j][1];
                fetch(i + DG_HRING - 1);
                asm volatile("cp.async.wait_group %0;\n" ::"n"(DG_HRING - 1) : "memory");      // this turn's values are here
                const bool stage_free = i < DG_STAGES || dg_wait(dg_smem(&empty[s]), ((i / DG_STAGES) & 1) ^ 1);
                uint4 packed = zero;
                if (on) {
                    const float4 h0 = *reinterpret_cast<const float4*>(mine + (i % DG_HRING) * (128 * 32));
                    const float4 h1 = *reinterpret_cast<const float4*>(mine + (i % DG_HRING) * (128 * 32) + 16);
                    ss = fmaf(h0.x, h0.x, ss); ss = fmaf(h0.y, h0.y, ss); ss = fmaf(h0.z, h0.z, ss); ss = fmaf(h0.w, h0.w, ss);
                    ss = fmaf(h1.x, h1.x, ss); ss = fmaf(h1.y, h1.y, ss); ss = fmaf(h1.z, h1.z, ss); ss = fmaf(h1.w, h1.w, ss);
                    __nv_bfloat162 a = __floats2bfloat162_rn(h0.x * g0.x, h0.y * g0.y), b = __floats2bfloat162_rn(h0.z * g0.z, h0.w * g0.w);
                    __nv_bfloat162 c = __floats2bfloat162_rn(h1.x * g1.x, h1.y * g1.y), d = __floats2bfloat162_rn(h1.z * g1.z, h1.w * g1.w);
                    packed = make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b),
                                        *reinterpret_cast<uint32_t*>(&c), *reinterpret_cast<uint32_t*>(&d));
                }
                fetch_g(i + DG_HRING, gq[j]);              // this slot's next use is DG_HRING turns away
                if (row_on && stage_free)                  // K-major tile, 128-byte swizzle: piece ^ (row % 8)
                    *reinterpret_cast<uint4*>(tiles + s * STAGE_BYTES + DG_W_BYTES + row * 128 + ((piece ^ (row & 7)) << 4)) = packed;
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                // the 128 threads meet once per tile and agree on whether every one of them got the stage in time
                uint32_t all_free;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.u32 p, %1, 0;\n\t"
                    "bar.red.and.pred q, 1, 128, p;\n\t"
                    "selp.u32 %0, 1, 0, q;\n\t}\n"
                    : "=r"(all_free) : "r"((uint32_t)stage_free) : "memory");
                if (!all_free) { *failed = 1; stop = true; break; }
                if (t == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(dg_smem(&full[s])) : "memory");
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (piece == 0) ss_part[row] = ss;
    }
    __syncwarp();

    if (REDUCE) {
        // ---- the partial tile -> shared memory as [batch row][32 outputs] per warp -> TMA reduce-add into Y.
        // A thread holds one output (weight row) for all batch rows; for each batch row the warp's 32 values
        // are neighbours in memory.  TMA clips batch rows >= M and outputs >= N. ----
        if (warp >= 2) {
            const bool good = k_iters == 0 || dg_wait(dg_smem(acc_full), 0, true);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int quarter = warp & 3;
            const int col = n0 + quarter * 32 + lane;
            float* piece = reinterpret_cast<float*>(tiles) + quarter * MP * 32;
            if (good && k_iters > 0 && n0 + quarter * 32 < N) {
                const float bv = (bias != nullptr && rank == 0 && col < N) ? bias[col] : 0.f;
#pragma unroll
                for (int c = 0; c < MP; c += 32) {
                    float v[32];
                    dg_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; ++j) piece[(c + j) * 32 + lane] = v[j] + bv;
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (k_splits == 1 && !accumulate)      // the only share of a result that is not added to: a store
                        asm volatile(
                            "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                            ::"l"(&map_y), "r"(n0 + quarter * 32), "r"(0), "r"(dg_smem(piece)) : "memory");
                    else
                    asm volatile(
                        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];\n"
                        ::"l"(&map_y), "r"(n0 + quarter * 32), "r"(0), "r"(dg_smem(piece)) : "memory");
                    asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
                }
            }
            if (!good) *failed = 1;
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0 && *failed && status) atomicOr(status, 2);
        if (warp == 1) {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)MP)
                         : "memory");
        }
        return;
    }

    // ---- the accumulator -> shared memory (all stages are free once it is complete) ----
    bool good = true;
    if (warp >= 2) {
        good = k_iters == 0 || dg_wait(dg_smem(acc_full), 0, true);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // weight row of this thread within the tile
#pragma unroll
        for (int c = 0; c < MP; c += 32) {
            float v[32];
            if (good && k_iters > 0) {
                dg_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) red[row * RED_LD + c + j] = v[j];
        }
        if (!good) *failed = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    if (n_ranks > 1) cluster.sync(); else __syncthreads();

    {
        // The (batch row, output column) pairs are dealt to the cluster's blocks in runs of 32 columns, so
        // every block adds and writes a share; each pair's partial sums are added in rank order.
        const float* peers[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) peers[p] = p < n_ranks ? cluster.map_shared_rank(red, p) : red;
        const float* peer_ss[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) peer_ss[p] = (NORM && p < n_ranks) ? cluster.map_shared_rank(ss_part, p) : ss_part;
        const int runs = (OUT_COLS / 32) * M;
        const int step = n_ranks * (DG_THREADS / 32);
        // four runs per turn: all their (remote) reads are in flight before the first sum
        for (int q0 = rank + n_ranks * (threadIdx.x >> 5); q0 < runs; q0 += 4 * step) {
            float pv[4][8], pu[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * step;
                const int m = q / (OUT_COLS / 32), c = (q - m * (OUT_COLS / 32)) * 32 + lane;
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    const bool on = q < runs && p < n_ranks;
                    pv[u][p] = on ? peers[p][c * RED_LD + m] : 0.f;
                    pu[u][p] = (SWIGLU && on) ? peers[p][(c + OUT_COLS) * RED_LD + m] : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int q = q0 + u * step;
                if (q >= runs) continue;
                const int m = q / (OUT_COLS / 32), c = (q - m * (OUT_COLS / 32)) * 32 + lane;
                const int col = n0 + c;
                float v = pv[u][0], w = pu[u][0];
#pragma unroll
                for (int p = 1; p < 8; ++p) { v += pv[u][p]; w += pu[u][p]; }
                if (col >= N) continue;
                if (NORM) {
                    float q2 = peer_ss[0][m];
#pragma unroll
                    for (int p = 1; p < 8; ++p) q2 += p < n_ranks ? peer_ss[p][m] : 0.f;
                    const float rms = sqrtf(q2 / (float)K + eps);
                    v /= rms;
                    if (SWIGLU) w /= rms;
                }
                if (bias) { v += bias[col]; if (SWIGLU) w += bias[col + N]; }
                if (SWIGLU)            // (a bfloat16 result keeps 8 bits: the fast exponential and division do)
                    v = sizeof(TO) == 2 ? __fdividef(v, 1.f + __expf(-v)) * w : (v / (1.f + expf(-v))) * w;
                TO* y = Y + (size_t)m * ldy + col;
                if (accumulate) v += to_f32<TO>(*y);
                *y = from_f32<TO>(v);
            }
        }
    }
    if (n_ranks > 1) cluster.sync(); else __syncthreads();   // peers keep their shared memory until it was read
    if (threadIdx.x == 0 && *failed && status) atomicOr(status, 2);
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)MP)
                     : "memory");
    }
}

static int dg_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {DG_BK, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}


// The REDUCE form: tiles x splits independent blocks, partial tiles summed into Y by TMA.
template <int MP>
static int dg_launch_reduce(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, float* Y, int M, int N,
                            int K, int ldy, int accumulate, int* status, int splits, cudaStream_t stream) {
    constexpr int STAGES = 4;
    constexpr int STAGE_BYTES = DG_W_BYTES + MP * DG_BK * 2;
    constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(4 * MP * 32 * 4 <= STAGES * STAGE_BYTES, "the partial tile must fit in the stages");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_gemm_tc_kernel<MP, false, float, STAGES, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    CUtensorMap my;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)ldy * 4};
        const cuuint32_t box[2] = {32, (cuuint32_t)MP};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = cuTensorMapEncodeTiled(&my, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, Y, dims, strides, box, estr,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return 1000 + (int)r;
    }
    if (!accumulate && splits > 1) {                      // several shares are added into a cleared result
        cudaError_t e = cudaMemset2DAsync(Y, (size_t)ldy * 4, 0, (size_t)N * 4, (size_t)M, stream);
        if (e != cudaSuccess) return (int)e;
    }
    const int tiles = (N + DG_ROWS - 1) / DG_ROWS;
    return tq_launch_pdl(TQ_PDL_DECODE_GEMM, decode_gemm_tc_kernel<MP, false, float, STAGES, true>, dim3(tiles * splits), dim3(DG_THREADS),
                         SMEM, stream, mw, mx, my, bias, Y, M, N, K, ldy, accumulate, splits, status, (const float*)nullptr, 0,
                         (const float*)nullptr, 0.f);
}

template <int MP, bool SWIGLU, typename TO, int DG_STAGES, bool NORM = false>
static int dg_launch_s(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* Y, int M, int N, int K,
                       int ldy, int accumulate, int* status, int ranks, cudaStream_t stream, const float* H = nullptr,
                       int ldh = 0, const float* G = nullptr, float eps = 0.f) {
    constexpr int STAGE_BYTES = DG_W_BYTES + MP * DG_BK * 2;
    constexpr int SMEM = DG_STAGES * STAGE_BYTES + 1024 + 256 + (NORM ? DG_HRING * 128 * 32 : 0);
    static_assert(DG_ROWS * (MP + 1) * 4 <= DG_STAGES * STAGE_BYTES, "partial sums must fit in the stages");
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(decode_gemm_tc_kernel<MP, SWIGLU, TO, DG_STAGES, false, NORM>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    constexpr int OUT_COLS = SWIGLU ? DG_ROWS / 2 : DG_ROWS;
    const int tiles = (N + OUT_COLS - 1) / OUT_COLS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * ranks, 1, 1);
    cfg.blockDim = dim3(DG_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = tq_pdl_enabled(TQ_PDL_DECODE_GEMM) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_gemm_tc_kernel<MP, SWIGLU, TO, DG_STAGES, false, NORM>, mw, mx,
                                       mw /* no map of Y in this form */, bias, (TO*)Y, M, N, K, ldy, accumulate, 1,
                                       status, H, ldh, G, eps);
    if (e != cudaSuccess) return (int)e;
    return tq_launch_status();
}

// Independent shares of K that a float32 product without gating is cut into (1: none; see dg_launch).
static int dg_reduce_shares(int N, int K) {
    const int tiles = (N + DG_ROWS - 1) / DG_ROWS, k_total = (K + DG_BK - 1) / DG_BK;
    // As many shares as fill the block slots once, down to two steps of 64 each (one where K is short).  Measured
    // alone in a replayed graph: shares of 8 steps against 2 cost the 7B shape's o product 7.9 against 7.1 us, a
    // 2048 x 2048 one 5.5 against 4.3, 896 x 4864 5.8 against 4.5.  (The cluster form's exchange through shared
    // memory costs a small product more than its whole main loop: 64 rows, 896 x 896, 26 us there and 4 us here.)
    if (k_total < 4 || tq_deterministic()) return 1;
    const int per_share = k_total >= 24 ? 2 : 1;
    int splits = 2 * tq_sm_count() / tiles;
    if (splits > k_total / per_share) splits = k_total / per_share;
    return splits > 1 ? splits : 1;
}

// Whether tq_decode_gemm_tc() would cut this float32 product into independent shares of K that are added into
// the result, which it therefore clears first unless told to accumulate.  A caller that keeps a zeroed buffer
// can then ask for accumulation and save the clearing.
TQ_API int tq_decode_gemm_tc_adds_shares(int N, int K) { return dg_reduce_shares(N, K) > 1 ? 1 : 0; }

template <int MP, bool SWIGLU, typename TO>
static int dg_launch(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* Y, int M, int N, int K,
                     int ldy, int accumulate, int* status, cudaStream_t stream) {
    constexpr int OUT_COLS = SWIGLU ? DG_ROWS / 2 : DG_ROWS;
    const int tiles = (N + OUT_COLS - 1) / OUT_COLS;
    const int k_total = (K + DG_BK - 1) / DG_BK;
    // Float32 results without gating: where the tiles do not fill the GPU's block slots (two per SM), independent
    // shares of K, as many as still run in one wave (dg_reduce_shares).  These results leave through TMA (a store for a single share that is not added to anything,
    // else a reduce-add), which costs a block far less than the exchange and the element-wise stores of the
    // cluster form below.  Y must be fit for TMA (16-byte aligned base and row stride).
    if (!SWIGLU && sizeof(TO) == 4 && (reinterpret_cast<uintptr_t>(Y) & 15) == 0 && (ldy & 3) == 0)
        return dg_launch_reduce<MP>(mw, mx, bias, (float*)Y, M, N, K, ldy, accumulate, status, dg_reduce_shares(N, K),
                                    stream);
    // split K while the grid is small and the shares stay long.  Measured best on the 7B shapes: up to 4
    // blocks and about 64 blocks in all for batches over 16 rows, up to 8 and a full GPU for smaller ones.
    const int max_ranks = M > 16 ? 4 : 8, want_blocks = M > 16 ? 64 : tq_sm_count();
    int ranks = 1;
    while (ranks < max_ranks && tiles * ranks < want_blocks && k_total / (ranks * 2) >= 4) ranks *= 2;
    return dg_launch_s<MP, SWIGLU, TO, 4>(mw, mx, bias, Y, M, N, K, ldy, accumulate, status, ranks, stream);
}

// X [M <= 64, K] and W [N, K] (or [2N, K] with swiglu) bfloat16, row strides
// ldx / ldw elements (multiples of 8, bases 16-byte aligned); Y [M, N]
// float32 or bfloat16 (accumulate needs float32).
TQ_API int tq_decode_gemm_tc(const void* X, const void* W, const float* bias, void* Y, int y_dtype, int M, int N, int K,
                             int ldx, int ldw, int ldy, int accumulate, int swiglu, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7)) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
        return (int)cudaErrorInvalidValue;
    if (accumulate && y_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    const int mp = M <= 32 ? 32 : 64;
    CUtensorMap mw, mx;
    int st = dg_make_map(&mw, W, swiglu ? 2ull * N : (uint64_t)N, (uint64_t)K, (uint64_t)ldw,
                         swiglu ? DG_ROWS / 2 : DG_ROWS);
    if (st) return st;
    st = dg_make_map(&mx, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, mp);
    if (st) return st;
#define TQ_DG(MP, S, T) return dg_launch<MP, S, T>(mw, mx, bias, Y, M, N, K, ldy, accumulate, status, stream)
    if (mp == 32) {
        if (swiglu && y_dtype == TQ_BF16) TQ_DG(32, true, bf16);
        if (swiglu && y_dtype == TQ_F32) TQ_DG(32, true, float);
        if (!swiglu && y_dtype == TQ_BF16) TQ_DG(32, false, bf16);
        if (!swiglu && y_dtype == TQ_F32) TQ_DG(32, false, float);
    } else {
        if (swiglu && y_dtype == TQ_BF16) TQ_DG(64, true, bf16);
        if (swiglu && y_dtype == TQ_F32) TQ_DG(64, true, float);
        if (!swiglu && y_dtype == TQ_BF16) TQ_DG(64, false, bf16);
        if (!swiglu && y_dtype == TQ_F32) TQ_DG(64, false, float);
    }
#undef TQ_DG
    return (int)cudaErrorInvalidValue;
}

// The same product with an RMS norm folded in (see NORM at the kernel): H [M <= 16, K] is the float32 residual
// stream (row stride ldh, a multiple of 4; base 16-byte aligned), G [K] the norm's float32 weights.  K is split
// over a thread-block cluster as in the plain form.
TQ_API int tq_decode_gemm_tc_norm(const float* H, const float* G, float eps, const void* W, const float* bias, void* Y,
                                  int y_dtype, int M, int N, int K, int ldh, int ldw, int ldy, int accumulate,
                                  int swiglu, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > DG_NORM_ROWS || K <= 0 || (K & 7) || (ldh & 3) || (ldw & 7) || !G || !H) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(H) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
        (reinterpret_cast<uintptr_t>(G) & 15))
        return (int)cudaErrorInvalidValue;
    if (accumulate && y_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    CUtensorMap mw;
    int st = dg_make_map(&mw, W, swiglu ? 2ull * N : (uint64_t)N, (uint64_t)K, (uint64_t)ldw,
                         swiglu ? DG_ROWS / 2 : DG_ROWS);
    if (st) return st;
    const int out_cols = swiglu ? DG_ROWS / 2 : DG_ROWS;
    const int tiles = (N + out_cols - 1) / out_cols, k_total = (K + DG_BK - 1) / DG_BK;
    int ranks = 1;
    while (ranks < 8 && tiles * ranks < tq_sm_count() && k_total / (ranks * 2) >= 4) ranks *= 2;
#define TQ_DGN(S, T) \
    return dg_launch_s<32, S, T, 4, true>(mw, mw, bias, Y, M, N, K, ldy, accumulate, status, ranks, stream, H, ldh, G, eps)
    if (swiglu && y_dtype == TQ_BF16) TQ_DGN(true, bf16);
    if (swiglu && y_dtype == TQ_F32) TQ_DGN(true, float);
    if (!swiglu && y_dtype == TQ_BF16) TQ_DGN(false, bf16);
    if (!swiglu && y_dtype == TQ_F32) TQ_DGN(false, float);
#undef TQ_DGN
    return (int)cudaErrorInvalidValue;
}
