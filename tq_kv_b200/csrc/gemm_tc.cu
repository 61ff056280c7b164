// Matrix product on the 5th-generation tensor cores of sm_100a:
//   C[M,N] = A[M,K] · B[N,K]^T     (bfloat16 operands, float32 accumulation)
// with tcgen05.mma issued by one thread, operands brought into shared memory
// by TMA (cp.async.bulk.tensor, 128-byte swizzle) through a 4-stage mbarrier
// pipeline, the accumulator in tensor memory (TMEM) and read back with
// tcgen05.ld for the epilogue.  One block computes one 128 x 256 tile.
//
// Epilogues (fused, float32): plain store (float32 or bfloat16, optional
// bias), accumulate into a float32 C (the residual sum,
// src/models/turbo_generic.rs:1969,1980), and SwiGLU gating
// (src/models/turbo_generic.rs:105-110): B then holds the gate rows followed
// by the up rows, a tile's 256 accumulator columns are 128 gate columns and
// the 128 up columns of the same outputs, and silu(gate) * up is written.
//
// Roles: warp 0 lane 0 issues TMA loads, warp 1 lane 0 issues the MMAs,
// warp 2 allocates and frees TMEM, all four warps run the epilogue (warp w
// reads TMEM lanes 32w .. 32w+31).  Every wait on an mbarrier is bounded:
// when a bound is hit the block raises a bit in *status, stops issuing work,
// still frees its TMEM and returns, so the host sees an error, not a hang.
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BN 256
#define TC_BK 64
#define TC_STAGES 4
#define TC_THREADS 128
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_B_BYTES (TC_BN * TC_BK * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */)
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

// ---- the kernel -------------------------------------------------------------------
// b_rows_second: SwiGLU only — row offset of the up rows in B (the number of outputs).
template <int EPI, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const float* __restrict__ bias, TO* __restrict__ C, int M, int N, int K, int ldc, int b_rows_second,
               int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    // bars[0..S): full, bars[S..2S): empty, bars[2S]: accumulator ready; then the TMEM address and a failure flag
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 1);
    volatile uint32_t* failed = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TC_BM;
    // output columns of this tile; with SwiGLU a tile yields 128 outputs from 128 gate + 128 up rows of B
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const int n0 = blockIdx.x * OUT_COLS;
    const int k_iters = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[TC_STAGES + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * TC_STAGES]), 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TC_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads ----
        for (int i = 0; i < k_iters; ++i) {
            const int s = i % TC_STAGES;
            if (!mbar_wait(smem_u32(&bars[TC_STAGES + s]), ((i / TC_STAGES) & 1) ^ 1)) { *failed = 1; break; }
            const uint32_t full = smem_u32(&bars[s]);
            const uint32_t a_dst = smem_u32(tiles + s * TC_STAGE_BYTES);
            const uint32_t b_dst = a_dst + TC_A_BYTES;
            mbar_expect_tx(full, TC_STAGE_BYTES);
            tma_load_2d(a_dst, &map_a, i * TC_BK, m0, full);
            if (EPI == EPI_SWIGLU) {
                tma_load_2d(b_dst, &map_b, i * TC_BK, n0, full);                                  // 128 gate rows
                tma_load_2d(b_dst + TC_B_BYTES / 2, &map_b, i * TC_BK, b_rows_second + n0, full); // 128 up rows
            } else {
                tma_load_2d(b_dst, &map_b, i * TC_BK, n0, full);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        const uint32_t idesc = instr_desc(TC_BM, TC_BN);
        bool ok = true;
        for (int i = 0; i < k_iters && ok; ++i) {
            const int s = i % TC_STAGES;
            if (!mbar_wait(smem_u32(&bars[s]), (i / TC_STAGES) & 1)) { *failed = 1; ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(tiles + s * TC_STAGE_BYTES);
            const uint32_t b_addr = a_addr + TC_A_BYTES;
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                // 16 elements of K = 32 bytes further inside the swizzle atom
                tc_mma(tmem_base, smem_desc_sw128(a_addr + k * 32), smem_desc_sw128(b_addr + k * 32), idesc,
                       (i > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(smem_u32(&bars[TC_STAGES + s]));          // frees the stage when these MMAs are done
        }
        tc_commit(smem_u32(&bars[2 * TC_STAGES]));              // accumulator ready (arrives even after a failure)
    }
    __syncwarp();

    // ---- epilogue: every warp reads its 32 TMEM lanes = 32 rows of the tile ----
    const bool acc_ok = mbar_wait(smem_u32(&bars[2 * TC_STAGES]), 0, true);
    tc_fence_after();
    __syncthreads();                                              // *failed is final
    const bool good = acc_ok && *failed == 0;
    if (good) {
        const int row = m0 + warp * 32 + lane;
        const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
        if (EPI == EPI_SWIGLU) {
#pragma unroll 1
            for (int c = 0; c < TC_BN / 2; c += 32) {
                float g[32], u[32];
                tc_ld32(t_row + c, g);
                tc_ld32(t_row + TC_BN / 2 + c, u);
                tc_wait_ld();
                if (row < M) {
                    TO* out = C + (size_t)row * ldc + n0 + c;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        if (n0 + c + j + 1 < N) {
                            const float a = (g[j] / (1.f + expf(-g[j]))) * u[j];
                            const float b = (g[j + 1] / (1.f + expf(-g[j + 1]))) * u[j + 1];
                            store2_f32<TO>(out + j, a, b);
                        } else if (n0 + c + j < N) {
                            out[j] = from_f32<TO>((g[j] / (1.f + expf(-g[j]))) * u[j]);
                        }
                    }
                }
            }
        } else {
#pragma unroll 1
            for (int c = 0; c < TC_BN; c += 32) {
                float v[32];
                tc_ld32(t_row + c, v);
                tc_wait_ld();
                if (row < M) {
                    TO* out = C + (size_t)row * ldc + n0 + c;
                    if (bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c + j < N) v[j] += bias[n0 + c + j];
                    }
                    const bool whole = n0 + c + 32 <= N && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
                    if (whole && sizeof(TO) == 4) {
                        float4* o4 = reinterpret_cast<float4*>(out);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float4 x = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                            if (EPI == EPI_ACCUM) {
                                const float4 old = o4[j];
                                x.x += old.x; x.y += old.y; x.z += old.z; x.w += old.w;
                            }
                            o4[j] = x;
                        }
                    } else if (whole) {
                        uint4* o4 = reinterpret_cast<uint4*>(out);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                            __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                            __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                            o4[j] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                               *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (n0 + c + j < N) {
                                float x = v[j];
                                if (EPI == EPI_ACCUM) x += to_f32<TO>(out[j]);
                                out[j] = from_f32<TO>(x);
                            }
                        }
                    }
                }
            }
        }
    } else if (threadIdx.x == 0 && status) {
        atomicOr(status, 2);                                      // a wait ran out: the result is not valid
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"((uint32_t)TC_BN)
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

template <int EPI, typename TO>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const float* bias, void* C, int M, int N, int K,
                     int ldc, int b_rows_second, int* status, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             TC_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    constexpr int OUT_COLS = EPI == EPI_SWIGLU ? TC_BN / 2 : TC_BN;
    const dim3 grid((N + OUT_COLS - 1) / OUT_COLS, (M + TC_BM - 1) / TC_BM);
    gemm_tc_kernel<EPI, TO><<<grid, TC_THREADS, TC_SMEM_BYTES, stream>>>(ma, mb, bias, (TO*)C, M, N, K, ldc,
                                                                        b_rows_second, status);
    return tq_launch_status();
}

// A [M, K] and B [N, K] (or [2N, K] with epilogue 2) bfloat16 with row strides
// lda / ldb (elements, multiples of 8; bases 16-byte aligned); C [M, N] with
// row stride ldc, float32 or bfloat16 (epilogue 1 needs float32).
// status: device int, bit 1 is raised if a pipeline wait ran out.
TQ_API int tq_gemm_tc(const void* A, const void* B, const float* bias, void* C, int c_dtype, int M, int N, int K,
                      int lda, int ldb, int ldc, int epilogue, int* status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || (lda & 7) || (ldb & 7)) return (int)cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_ACCUM && c_dtype != TQ_F32) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && (N & 1)) return (int)cudaErrorInvalidValue;
    CUtensorMap ma, mb;
    int st = make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, TC_BM);
    if (st) return st;
    const uint64_t b_rows = epilogue == EPI_SWIGLU ? 2ull * N : (uint64_t)N;
    st = make_map(&mb, B, b_rows, (uint64_t)K, (uint64_t)ldb, epilogue == EPI_SWIGLU ? TC_BN / 2 : TC_BN);
    if (st) return st;
#define TQ_TC(E, T) return launch_tc<E, T>(ma, mb, bias, C, M, N, K, ldc, N, status, stream)
    if (epilogue == EPI_STORE && c_dtype == TQ_F32) TQ_TC(EPI_STORE, float);
    if (epilogue == EPI_STORE && c_dtype == TQ_BF16) TQ_TC(EPI_STORE, bf16);
    if (epilogue == EPI_ACCUM) TQ_TC(EPI_ACCUM, float);
    if (epilogue == EPI_SWIGLU && c_dtype == TQ_F32) TQ_TC(EPI_SWIGLU, float);
    if (epilogue == EPI_SWIGLU && c_dtype == TQ_BF16) TQ_TC(EPI_SWIGLU, bf16);
#undef TQ_TC
    return (int)cudaErrorInvalidValue;
}
