// Matrix products on CUDA cores with float32 fused multiply-adds (no tensor
// cores, no reduced-precision mode): C[M,N] = A[M,K] · W[N,K]^T (+ bias[N])
// (+ C).  W is row-major [out, in] as the checkpoints store it
// (src/models/turbo_generic.rs:68-91: forward = x · W^T).
//
//  * gemm_tiled: any M, N, K and any mix of float32 / bfloat16 operands; the
//    whole float32 path runs on it, and so do operands that the tensor-core
//    kernels refuse.
//  * gemv_rows: M <= 8 rows of A per pass, one warp per output column,
//    16-byte weight loads — the memory-bound shape of decoding.  Optional
//    SwiGLU pairing: W holds the gate rows then the up rows, and the kernel
//    writes silu(gate) * up.
#include "common.cuh"

#define GT_BM 64
#define GT_BN 64
#define GT_BK 16

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_tiled_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                  TO* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
    __shared__ float As[GT_BK][GT_BM + 4];
    __shared__ float Ws[GT_BK][GT_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GT_BM, n0 = blockIdx.x * GT_BN;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GT_BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread; consecutive threads walk k
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (m0 + r < M) a = to_f32<TA>(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) w = to_f32<TW>(W[(size_t)(n0 + r) * ldw + k]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GT_BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            TO* c = C + (size_t)m * ldc + n;
            if (accumulate) v += to_f32<TO>(*c);
            *c = from_f32<TO>(v);
        }
    }
}

TQ_API int tq_gemm_tiled(const void* A, int a_dtype, const void* W, int w_dtype, const float* bias, void* C,
                         int c_dtype, int M, int N, int K, int lda, int ldw, int ldc, int accumulate,
                         cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    const dim3 grid((N + GT_BN - 1) / GT_BN, (M + GT_BM - 1) / GT_BM);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define TQ_LAUNCH(TA, TW, TO)                                                                             \
    gemm_tiled_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, bias, (TO*)C, M, N, K, \
                                                            lda, ldw, ldc, accumulate)
    const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (code) {
        case 0: TQ_LAUNCH(float, float, float); break;
        case 1: TQ_LAUNCH(float, float, bf16); break;
        case 2: TQ_LAUNCH(float, bf16, float); break;
        case 3: TQ_LAUNCH(float, bf16, bf16); break;
        case 4: TQ_LAUNCH(bf16, float, float); break;
        case 5: TQ_LAUNCH(bf16, float, bf16); break;
        case 6: TQ_LAUNCH(bf16, bf16, float); break;
        case 7: TQ_LAUNCH(bf16, bf16, bf16); break;
        default: return (int)cudaErrorInvalidValue;
    }
#undef TQ_LAUNCH
    return tq_launch_status();
}

// ---------------------------------------------------------------------------
// gemv_rows: grid (ceil(N / warps), ceil(M / 8)); warp -> output column n.
// ---------------------------------------------------------------------------
#define GV_ROWS 8
#define GV_WARPS 4

template <typename TA, typename TW, typename TO, bool SWIGLU>
__global__ void __launch_bounds__(GV_WARPS * 32)
gemv_rows_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                 TO* __restrict__ C, int M, int N, int K, int lda, int ldw, int ldc, int accumulate) {
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * GV_WARPS + (threadIdx.x >> 5);
    if (n >= N) return;
    const int m0 = blockIdx.y * GV_ROWS;
    const int rows = min(GV_ROWS, M - m0);
    constexpr int VW = Vec16<TW>::N;
    const TW* w0 = W + (size_t)n * ldw;
    const TW* w1 = SWIGLU ? W + (size_t)(n + N) * ldw : nullptr;
    float acc0[GV_ROWS], acc1[GV_ROWS];
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }

    const bool vec_ok = (K % VW == 0) && (ldw % VW == 0) && (lda % VW == 0) &&
                        ((reinterpret_cast<uintptr_t>(W) & 15) == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
    if (vec_ok) {
        for (int k = lane * VW; k < K; k += 32 * VW) {
            float wv0[VW], wv1[VW];
            load16_f32<TW>(w0 + k, wv0);
            if (SWIGLU) load16_f32<TW>(w1 + k, wv1);
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) {
                if (r < rows) {
                    const TA* a = A + (size_t)(m0 + r) * lda + k;
                    float av[VW];
                    if (sizeof(TA) == sizeof(TW)) {
                        load16_f32<TA>(a, av);
                    } else {
#pragma unroll
                        for (int e = 0; e < VW; ++e) av[e] = to_f32<TA>(a[e]);
                    }
#pragma unroll
                    for (int e = 0; e < VW; ++e) {
                        acc0[r] = fmaf(av[e], wv0[e], acc0[r]);
                        if (SWIGLU) acc1[r] = fmaf(av[e], wv1[e], acc1[r]);
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv0 = to_f32<TW>(w0[k]);
            const float wv1 = SWIGLU ? to_f32<TW>(w1[k]) : 0.f;
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) {
                if (r < rows) {
                    const float av = to_f32<TA>(A[(size_t)(m0 + r) * lda + k]);
                    acc0[r] = fmaf(av, wv0, acc0[r]);
                    if (SWIGLU) acc1[r] = fmaf(av, wv1, acc1[r]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) {
        if (r < rows) {
            float v0 = warp_sum(acc0[r]);
            float v1 = SWIGLU ? warp_sum(acc1[r]) : 0.f;
            if (lane == 0) {
                if (bias) { v0 += bias[n]; if (SWIGLU) v1 += bias[n + N]; }
                float v = v0;
                if (SWIGLU) v = (v0 / (1.f + expf(-v0))) * v1;
                TO* c = C + (size_t)(m0 + r) * ldc + n;
                if (accumulate) v += to_f32<TO>(*c);
                *c = from_f32<TO>(v);
            }
        }
    }
}

// N is the number of output columns; with swiglu != 0, W has 2*N rows.
TQ_API int tq_gemv_rows(const void* A, int a_dtype, const void* W, int w_dtype, const float* bias, void* C,
                        int c_dtype, int M, int N, int K, int lda, int ldw, int ldc, int accumulate, int swiglu,
                        cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return (int)cudaErrorInvalidValue;
    const dim3 grid((N + GV_WARPS - 1) / GV_WARPS, (M + GV_ROWS - 1) / GV_ROWS);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define TQ_LAUNCH2(TA, TW, TO)                                                                                 \
    do {                                                                                                       \
        if (swiglu)                                                                                            \
            gemv_rows_kernel<TA, TW, TO, true><<<grid, GV_WARPS * 32, 0, stream>>>(                           \
                (const TA*)A, (const TW*)W, bias, (TO*)C, M, N, K, lda, ldw, ldc, accumulate);                 \
        else                                                                                                   \
            gemv_rows_kernel<TA, TW, TO, false><<<grid, GV_WARPS * 32, 0, stream>>>(                          \
                (const TA*)A, (const TW*)W, bias, (TO*)C, M, N, K, lda, ldw, ldc, accumulate);                 \
    } while (0)
    const int code = a_dtype * 4 + w_dtype * 2 + c_dtype;
    switch (code) {
        case 0: TQ_LAUNCH2(float, float, float); break;
        case 2: TQ_LAUNCH2(float, bf16, float); break;
        case 4: TQ_LAUNCH2(bf16, float, float); break;
        case 5: TQ_LAUNCH2(bf16, float, bf16); break;
        case 6: TQ_LAUNCH2(bf16, bf16, float); break;
        case 7: TQ_LAUNCH2(bf16, bf16, bf16); break;
        default: return (int)cudaErrorInvalidValue;
    }
#undef TQ_LAUNCH2
    return tq_launch_status();
}
