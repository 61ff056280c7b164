// Weight-streaming matrix product for decoding: Y[M,N] = X[M,K] · W[N,K]^T
// with M <= 64 rows of activations, bfloat16 operands, float32 accumulation
// on the tensor cores (mma.sync m16n8k16: W rows are the "M" side of the
// instruction, the batch is its "N" side).  The kernel is bound by reading W
// once from HBM; everything is arranged so that each lane loads 16 contiguous
// bytes of a W row and many such loads are in flight.
//
// Work split: a block owns 16 (or 32) output columns, its 8 warps split K and
// add their partial sums through shared memory in warp order.  Where that
// gives too few blocks to fill the GPU (few columns, long K), a thread-block
// cluster of 2, 4 or 8 blocks splits K once more and the cluster's first
// block adds the others' sums, read from their shared memory in rank order.
// So the result never depends on scheduling.  Epilogues: bias, SwiGLU gating (W holds the
// gate rows, then the up rows: src/models/turbo_generic.rs:105-110), adding
// into the float32 residual stream (:1969, :1980), float32 or bfloat16 output.
//
// The k index inside a 32-wide block is permuted the same way for both
// operands (lane tid4 owns k = 8*tid4 .. 8*tid4+7 and feeds elements 0..3 to
// one mma and 4..7 to the next), which leaves every dot product unchanged.
#include "common.cuh"
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define SK_WARPS 8

__device__ __forceinline__ void mma_bf16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    // not volatile: the weights are read-only, so the compiler may hoist these loads ahead of the math
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// NT: tiles of 8 batch rows (M <= 8*NT).  TW: W row tiles of 16 per warp (1 or 2).
// SWIGLU: TW must be 2; tile 0 = gate rows n, tile 1 = up rows n + N.
//
// NORM: the activations are not given as bfloat16 rows but as the float32 residual stream H [M, K] with the
// weights G [K] of an RMS norm (src/models/turbo_generic.rs:41-51): the kernel multiplies with
// x = bfloat16(h * g) and scales each batch row's sums by 1 / sqrt(mean(h^2) + eps) before the epilogue, so
// that the norm needs no kernel and no trip through memory of its own.  The sums of squares are gathered
// beside the partial products (every k is read by exactly one lane of one warp of one block of the cluster).
template <int NT, int TW, bool SWIGLU, typename TO, bool NORM>
__global__ void __launch_bounds__(SK_WARPS * 32)
skinny_gemm_kernel(const void* __restrict__ Xv, const bf16* __restrict__ W, const float* __restrict__ bias,
                   TO* __restrict__ Y, int M, int N, int K, int ldx, int ldw, int ldy, int accumulate,
                   const float* __restrict__ G, float eps) {
    constexpr int COLS = SWIGLU ? 16 : 16 * TW;          // output columns of this block
    constexpr int PER_WARP = TW * 16 * (8 * NT + 1);
    extern __shared__ float red_raw[];
    float (*red)[TW][16][8 * NT + 1] = reinterpret_cast<float (*)[TW][16][8 * NT + 1]>(red_raw);
    float* red_ss = red_raw + SK_WARPS * PER_WARP;       // NORM: [warp][batch row] sums of squares
    const bf16* X = reinterpret_cast<const bf16*>(Xv);
    const float* H = reinterpret_cast<const float*>(Xv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gid = lane >> 2, tid4 = lane & 3;
    cg::cluster_group cluster = cg::this_cluster();
    const int n_ranks = (int)cluster.num_blocks();       // blocks that share these columns and split K
    const int rank = (int)cluster.block_rank();
    const int col0 = (blockIdx.x / n_ranks) * COLS;

    // rows of W this lane reads (clamped; masked at the store)
    const bf16* wp[TW][2];
#pragma unroll
    for (int t = 0; t < TW; ++t) {
        const int base = SWIGLU ? (col0 + t * N) : (col0 + 16 * t);
        const int limit = SWIGLU ? (t + 1) * N : N;
        int r0 = base + gid, r1 = base + gid + 8;
        r0 = r0 < limit ? r0 : limit - 1;
        r1 = r1 < limit ? r1 : limit - 1;
        wp[t][0] = W + (size_t)r0 * ldw + tid4 * 8;
        wp[t][1] = W + (size_t)r1 * ldw + tid4 * 8;
    }
    const bf16* xp[NT];
    bool xv[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int m = n * 8 + gid;
        xv[n] = m < M;
        xp[n] = X + (size_t)(xv[n] ? m : 0) * ldx + tid4 * 8;
    }
    const float* hp[NT];
    float ss[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        hp[n] = H + (size_t)(xv[n] ? n * 8 + gid : 0) * ldx + tid4 * 8;
        ss[n] = 0.f;
    }
    // NORM: eight values of row n at k-block offset k as bfloat16(h * g); their squares are added to ss[n]
    auto normed8 = [&](int n, int k) -> uint4 {
        if (!xv[n]) return make_uint4(0, 0, 0, 0);
        const float4 h0 = *reinterpret_cast<const float4*>(hp[n] + k), h1 = *reinterpret_cast<const float4*>(hp[n] + k + 4);
        const float4 g0 = *reinterpret_cast<const float4*>(G + k + tid4 * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(G + k + tid4 * 8 + 4);
        ss[n] = fmaf(h0.x, h0.x, ss[n]); ss[n] = fmaf(h0.y, h0.y, ss[n]); ss[n] = fmaf(h0.z, h0.z, ss[n]);
        ss[n] = fmaf(h0.w, h0.w, ss[n]); ss[n] = fmaf(h1.x, h1.x, ss[n]); ss[n] = fmaf(h1.y, h1.y, ss[n]);
        ss[n] = fmaf(h1.z, h1.z, ss[n]); ss[n] = fmaf(h1.w, h1.w, ss[n]);
        __nv_bfloat162 a = __floats2bfloat162_rn(h0.x * g0.x, h0.y * g0.y), b = __floats2bfloat162_rn(h0.z * g0.z, h0.w * g0.w);
        __nv_bfloat162 c = __floats2bfloat162_rn(h1.x * g1.x, h1.y * g1.y), d = __floats2bfloat162_rn(h1.z * g1.z, h1.w * g1.w);
        return make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b),
                          *reinterpret_cast<uint32_t*>(&c), *reinterpret_cast<uint32_t*>(&d));
    };
    float acc[TW][NT][4];
#pragma unroll
    for (int t = 0; t < TW; ++t)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][n][i] = 0.f;

    const int kblocks = K >> 5;
    const int parts = SK_WARPS * n_ranks;
    const int per = (kblocks + parts - 1) / parts;
    const int kb0 = min(kblocks, (rank * SK_WARPS + warp) * per);
    const int kb1 = min(kblocks, kb0 + per);
    // U k-blocks per turn: all their weight loads are issued before the first mma needs one.  The first
    // turn's loads are issued before this kernel waits for its predecessor: weights do not depend on it.
    constexpr int U = (NT <= 2) ? 4 : 2;
    uint4 a[U][TW][2];
    auto load_weights = [&](int kb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const bool on = kb + u < kb1;
            const int k = (on ? kb + u : kb0) << 5;
#pragma unroll
            for (int t = 0; t < TW; ++t) {
                a[u][t][0] = ld_stream16(wp[t][0] + k);
                a[u][t][1] = ld_stream16(wp[t][1] + k);
                if (!on) a[u][t][0] = a[u][t][1] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    if (kb0 < kb1) load_weights(kb0);
    pdl_wait();                                            // the activations are ready from here on
    pdl_launch();
    for (int kb = kb0; kb < kb1; kb += U) {
        if (kb > kb0) load_weights(kb);
        uint4 bx[U][NT <= 2 ? NT : 1];
        if (NT <= 2) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = (kb + u < kb1 ? kb + u : kb0) << 5;
#pragma unroll
                for (int n = 0; n < (NT <= 2 ? NT : 1); ++n) {
                    if (NORM) bx[u][n] = (kb + u < kb1) ? normed8(n, k) : make_uint4(0, 0, 0, 0);
                    else bx[u][n] = xv[n] ? *reinterpret_cast<const uint4*>(xp[n] + k) : make_uint4(0, 0, 0, 0);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb + u < kb1 ? kb + u : kb0) << 5;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                uint4 b;
                if (NT <= 2) b = bx[u][n < 2 ? n : 0];
                else if (NORM) b = (kb + u < kb1) ? normed8(n, k) : make_uint4(0, 0, 0, 0);
                else b = xv[n] ? *reinterpret_cast<const uint4*>(xp[n] + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int t = 0; t < TW; ++t) {
                    mma_bf16_16816(acc[t][n], a[u][t][0].x, a[u][t][1].x, a[u][t][0].y, a[u][t][1].y, b.x, b.y);
                    mma_bf16_16816(acc[t][n], a[u][t][0].z, a[u][t][1].z, a[u][t][0].w, a[u][t][1].w, b.z, b.w);
                }
            }
        }
    }
    // partial sums of this warp: c0,c1 -> (row gid, batch 2*tid4, +1); c2,c3 -> (row gid+8, same)
#pragma unroll
    for (int t = 0; t < TW; ++t)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            red[warp][t][gid][n * 8 + 2 * tid4] = acc[t][n][0];
            red[warp][t][gid][n * 8 + 2 * tid4 + 1] = acc[t][n][1];
            red[warp][t][gid + 8][n * 8 + 2 * tid4] = acc[t][n][2];
            red[warp][t][gid + 8][n * 8 + 2 * tid4 + 1] = acc[t][n][3];
        }
    if (NORM) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {                     // the four lanes of a row hold its k in quarters
            float v = ss[n];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (tid4 == 0) red_ss[warp * 8 * NT + n * 8 + gid] = v;
        }
    }
    __syncthreads();
    // block sums: warps added in order into red[0]
    for (int e = threadIdx.x; e < PER_WARP; e += blockDim.x) {
        float v = red_raw[e];
#pragma unroll
        for (int w = 1; w < SK_WARPS; ++w) v += red_raw[w * PER_WARP + e];
        red_raw[e] = v;
    }
    if (NORM && threadIdx.x < 8 * NT) {
        float v = red_ss[threadIdx.x];
#pragma unroll
        for (int w = 1; w < SK_WARPS; ++w) v += red_ss[w * 8 * NT + threadIdx.x];
        red_ss[threadIdx.x] = v;
    }
    if (n_ranks > 1) cluster.sync(); else __syncthreads();
    if (rank == 0) {
        // one thread per (column, batch row): the cluster's blocks added in rank order, then the epilogue
        for (int e = threadIdx.x; e < COLS * 8 * NT; e += blockDim.x) {
            const int m = e / COLS, c = e - m * COLS;      // consecutive threads -> consecutive columns
            if (m >= M) continue;
            const int col = col0 + c;
            if (col >= N) continue;
            const int t = SWIGLU ? 0 : (c >> 4), r = SWIGLU ? c : (c & 15);
            float v = red[0][t][r][m], u = SWIGLU ? red[0][TW - 1][r][m] : 0.f;
            for (int p = 1; p < n_ranks; ++p) {
                const float* peer = cluster.map_shared_rank(red_raw, p);
                v += peer[(t * 16 + r) * (8 * NT + 1) + m];
                if (SWIGLU) u += peer[((TW - 1) * 16 + r) * (8 * NT + 1) + m];
            }
            if (NORM) {
                float q = red_ss[m];
                for (int p = 1; p < n_ranks; ++p) q += cluster.map_shared_rank(red_raw, p)[SK_WARPS * PER_WARP + m];
                const float rms = sqrtf(q / (float)K + eps);
                v /= rms;
                if (SWIGLU) u /= rms;
            }
            if (bias) { v += bias[col]; if (SWIGLU) u += bias[col + N]; }
            if (SWIGLU)                // (a bfloat16 result keeps 8 bits: the fast exponential and division do)
                v = sizeof(TO) == 2 ? __fdividef(v, 1.f + __expf(-v)) * u : (v / (1.f + expf(-v))) * u;
            TO* y = Y + (size_t)m * ldy + col;
            if (accumulate) v += to_f32<TO>(*y);
            *y = from_f32<TO>(v);
        }
    }
    if (n_ranks > 1) cluster.sync();                       // peers keep their shared memory until it was read
}

template <int NT, int TW, bool SWIGLU, typename TO, bool NORM = false>
static int launch_skinny(const void* X, const bf16* W, const float* bias, void* Y, int M, int N, int K, int ldx,
                         int ldw, int ldy, int accumulate, cudaStream_t stream, const float* G = nullptr,
                         float eps = 0.f) {
    constexpr int COLS = SWIGLU ? 16 : 16 * TW;
    const int tiles = (N + COLS - 1) / COLS;
    // split K over a cluster while the grid is small and every warp keeps a few k-blocks
    int ranks = 1;
    while (ranks < 8 && tiles * ranks < 4 * tq_sm_count() && (K >> 5) / (SK_WARPS * ranks * 2) >= 4) ranks *= 2;
    constexpr size_t smem = sizeof(float) * (SK_WARPS * TW * 16 * (8 * NT + 1) + (NORM ? SK_WARPS * 8 * NT : 0));
    static bool configured = false;          // per template instance
    if (smem > 48 * 1024 && !configured) {
        cudaError_t e = cudaFuncSetAttribute(skinny_gemm_kernel<NT, TW, SWIGLU, TO, NORM>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * ranks, 1, 1);
    cfg.blockDim = dim3(SK_WARPS * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // see pdl_wait() in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = tq_pdl_enabled(TQ_PDL_SKINNY) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel<NT, TW, SWIGLU, TO, NORM>, X, W, bias, (TO*)Y, M, N, K,
                                       ldx, ldw, ldy, accumulate, G, eps);
    if (e != cudaSuccess) return (int)e;
    return tq_launch_status();
}

template <bool SWIGLU, typename TO>
static int dispatch_skinny(const bf16* X, const bf16* W, const float* bias, void* Y, int M, int N, int K, int ldx,
                           int ldw, int ldy, int accumulate, cudaStream_t s) {
    if (SWIGLU) {
        if (M <= 8) return launch_skinny<1, 2, true, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
        if (M <= 16) return launch_skinny<2, 2, true, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
        if (M <= 32) return launch_skinny<4, 2, true, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
        return launch_skinny<8, 2, true, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
    }
    if (M <= 8) return launch_skinny<1, 1, false, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
    if (M <= 16) return launch_skinny<2, 1, false, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
    if (M <= 32) return launch_skinny<4, 2, false, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
    return launch_skinny<8, 2, false, TO>(X, W, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, s);
}

// X [M, K] bf16, W [N, K] (or [2N, K] with swiglu) bf16, Y [M, N] float32 or
// bfloat16.  Needs M <= 64, K a multiple of 32, 16-byte aligned rows.
TQ_API int tq_skinny_gemm(const void* X, const void* W, const float* bias, void* Y, int y_dtype, int M, int N, int K,
                          int ldx, int ldw, int ldy, int accumulate, int swiglu, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K & 31) || (ldx & 7) || (ldw & 7)) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
        return (int)cudaErrorInvalidValue;
    if (accumulate && y_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    const bf16* x = (const bf16*)X;
    const bf16* w = (const bf16*)W;
    if (swiglu) {
        if (y_dtype == TQ_F32) return dispatch_skinny<true, float>(x, w, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        if (y_dtype == TQ_BF16) return dispatch_skinny<true, bf16>(x, w, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
    } else {
        if (y_dtype == TQ_F32) return dispatch_skinny<false, float>(x, w, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
        if (y_dtype == TQ_BF16) return dispatch_skinny<false, bf16>(x, w, bias, Y, M, N, K, ldx, ldw, ldy, accumulate, stream);
    }
    return (int)cudaErrorInvalidValue;
}

// The same with the RMS norm folded in (see NORM above): H [M <= 16, K] is the float32 residual stream with row
// stride ldh (a multiple of 4, base 16-byte aligned), G [K] the norm's float32 weights.
TQ_API int tq_skinny_gemm_norm(const float* H, const float* G, float eps, const void* W, const float* bias, void* Y,
                               int y_dtype, int M, int N, int K, int ldh, int ldw, int ldy, int accumulate, int swiglu,
                               cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K & 31) || (ldh & 3) || (ldw & 7) || !G) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(H) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
        (reinterpret_cast<uintptr_t>(G) & 15))
        return (int)cudaErrorInvalidValue;
    if (accumulate && y_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    const bf16* w = (const bf16*)W;
#define TQ_SKN(NT, TW, S, T) \
    return launch_skinny<NT, TW, S, T, true>(H, w, bias, Y, M, N, K, ldh, ldw, ldy, accumulate, stream, G, eps)
    if (swiglu) {
        if (y_dtype == TQ_F32) { if (M <= 8) TQ_SKN(1, 2, true, float); TQ_SKN(2, 2, true, float); }
        if (y_dtype == TQ_BF16) { if (M <= 8) TQ_SKN(1, 2, true, bf16); TQ_SKN(2, 2, true, bf16); }
    } else {
        if (y_dtype == TQ_F32) { if (M <= 8) TQ_SKN(1, 1, false, float); TQ_SKN(2, 1, false, float); }
        if (y_dtype == TQ_BF16) { if (M <= 8) TQ_SKN(1, 1, false, bf16); TQ_SKN(2, 1, false, bf16); }
    }
#undef TQ_SKN
    return (int)cudaErrorInvalidValue;
}
