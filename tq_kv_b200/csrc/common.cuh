// Shared helpers of the hand-written sm_100a kernels: element conversion,
// warp/block reductions, the C ABI conventions.
//
// Every exported function is `extern "C"`, takes raw device pointers and a
// cudaStream_t, launches on that stream and returns the launch's cudaError_t
// as an int (0 = success).  Sizes are validated by the Python wrappers, which
// raise before anything is launched; the functions re-check what would make
// a kernel read out of bounds and return cudaErrorInvalidValue instead of
// launching.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define TQ_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C ABI
#define TQ_F32 0
#define TQ_BF16 1

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Number of elements of T in a 16-byte vector.
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

// Loads 16 bytes of T from `p` (16-byte aligned) and widens to float.
template <typename T> __device__ __forceinline__ void load16_f32(const T* p, float* out);
template <> __device__ __forceinline__ void load16_f32<float>(const float* p, float* out) {
    float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <> __device__ __forceinline__ void load16_f32<bf16>(const bf16* p, float* out) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Loads two consecutive elements (4- or 8-byte aligned) and widens to float.
template <typename T> __device__ __forceinline__ float2 load2_f32(const T* p);
template <> __device__ __forceinline__ float2 load2_f32<float>(const float* p) {
    return *reinterpret_cast<const float2*>(p);
}
template <> __device__ __forceinline__ float2 load2_f32<bf16>(const bf16* p) {
    uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ void store2_f32(T* p, float a, float b);
template <> __device__ __forceinline__ void store2_f32<float>(float* p, float a, float b) {
    *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <> __device__ __forceinline__ void store2_f32<bf16>(bf16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a block of up to 1024 threads; `red` holds 32 floats of shared
// memory.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

static inline int tq_launch_status() { return (int)cudaGetLastError(); }

// Streaming multiprocessors of the current device (asked once per device): grids and splits are sized by it.
static inline int tq_sm_count() {
    static int counts[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!counts[dev]) {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        counts[dev] = sms > 0 ? sms : 1;
    }
    return counts[dev];
}

// TQ_DETERMINISTIC=1: no product is cut along K into shares that meet in memory in arrival order (the tcgen05
// products then run somewhat slower: fewer blocks where tiles are few).  Every sum is then made in a fixed
// order, and two runs of the same steps give the same bits.
static inline bool tq_deterministic() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("TQ_DETERMINISTIC");
        on = (e && e[0] == '1') ? 1 : 0;
    }
    return on == 1;
}

// ---- programmatic dependent launch -------------------------------------------
// Kernels of a decode step are short and run back to back.  Launched with
// this attribute, a kernel may start while its predecessor in the stream is
// still draining: it does whatever does not depend on the predecessor (index
// arithmetic, requesting its first weight tiles), then pdl_wait() blocks until
// the predecessor has completed and its writes are visible.  Every kernel
// launched this way calls pdl_wait() before it reads or writes anything a
// predecessor may touch, and pdl_launch() right after, which lets its own
// successor start early in turn.  Without the launch attribute both
// instructions do nothing.
//
// Measured on decode steps: together the families gain 3 to 9 % on the 7B
// shape and up to 14 % on the 0.5B shape, whose step is mostly launch latency.
// One thing loses: a kernel let in while the decode attention streams the
// cache (2 to 4 % of the step), whichever kernel that is; so flash_decode
// waits but never calls pdl_launch(), and the merge that follows it, which
// then has nothing to gain, is left out of the default.  TQ_PDL=0 switches it off,
// TQ_PDL=1 on for every family, a larger number is a mask of families:
// 2 element-wise, 4 skinny_gemm, 8 decode_gemm_tc, 16 flash_decode,
// 32 attention merge, 64 sampling, 128 the many-row product (gemm_tc), 256 the prompt attention.  Every launch
// names its family.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

#define TQ_PDL_ELEMENTWISE 2
#define TQ_PDL_SKINNY 4
#define TQ_PDL_DECODE_GEMM 8
#define TQ_PDL_FLASH_DECODE 16
#define TQ_PDL_MERGE 32
#define TQ_PDL_SAMPLING 64
#define TQ_PDL_GEMM_TC 128
#define TQ_PDL_PREFILL_ATTENTION 256
#define TQ_PDL_DEFAULT (TQ_PDL_ELEMENTWISE | TQ_PDL_SKINNY | TQ_PDL_DECODE_GEMM | TQ_PDL_FLASH_DECODE | TQ_PDL_SAMPLING | \
                        TQ_PDL_GEMM_TC | TQ_PDL_PREFILL_ATTENTION)
static inline bool tq_pdl_enabled(int family) {
    static int mask = -1;
    if (mask < 0) {
        const char* e = getenv("TQ_PDL");
        mask = e ? atoi(e) : TQ_PDL_DEFAULT;
        if (mask == 1) mask = 0x7fffffff;
        if (mask < 0) mask = 0;
    }
    return (mask & family) != 0;
}

template <typename... KArgs, typename... Args>
static inline int tq_launch_pdl(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = tq_pdl_enabled(family) ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
