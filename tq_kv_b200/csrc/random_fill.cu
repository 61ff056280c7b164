// Random weights on the device: out[i] = offset + std * z(key, i), z standard normal.
//
// The generator is counter-based: element i of a tensor depends on (key, i)
// only, where the key is made on the host from the seed and the tensor's name
// (weights/random_init.py).  Every floating-point step is a single IEEE
// float32 operation (add, multiply, divide, square root; never a fused
// multiply-add, never a library logarithm or cosine), written in the same
// order as the numpy twin in weights/random_init.py, so that host and device
// produce the same bits.  The reference has no random-weights mode.
//
// z = sqrt(-2 ln u1) * cos(2 pi u2)     (Box-Muller, cosine branch)
//   64 bits = mix(key ^ i * C): the top 24 bits k1 give u1 = (k1 + 1) / 2^24 in (0, 1],
//   the next 24 bits k2 give the angle k2 / 2^24 of a full turn.
//   ln u1: u1's exponent and mantissa are split by bit operations, the mantissa m is brought into
//          [1/sqrt 2, sqrt 2) and ln m = 2 (s + s^3/3 + ... + s^11/11) with s = (m - 1) / (m + 1).
//   cos:   the top three bits of k2 name the octant, the other 21 the place t in it; the angle inside the octant
//          (or its mirror image for odd octants) is at most pi/4, where the Taylor polynomials of sine (to x^9)
//          and cosine (to x^10) are exact to float32 rounding.
#include "common.cuh"

__device__ __forceinline__ unsigned long long rf_mix(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float rf_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float rf_add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ float rf_normal(unsigned long long key, unsigned long long i) {
    const unsigned long long bits = rf_mix(key ^ (i * 0xD6E8FEB86659FD93ull));
    const unsigned int k1 = (unsigned int)(bits >> 40), k2 = (unsigned int)(bits >> 16) & 0xFFFFFFu;

    // ---- ln u1, u1 = (k1 + 1) / 2^24
    const unsigned int fb = __float_as_uint((float)(k1 + 1));           // an integer up to 2^24: exact
    int e = (int)(fb >> 23) - 127;
    float m = __uint_as_float((fb & 0x7FFFFFu) | 0x3F800000u);         // [1, 2)
    if (m > 0x1.6a09e6p+0f) { m = rf_mul(m, 0.5f); e += 1; }
    const float s = __fdiv_rn(rf_add(m, -1.0f), rf_add(m, 1.0f));
    const float s2 = rf_mul(s, s);
    float p = 1.0f / 11.0f;
    p = rf_add(rf_mul(p, s2), 1.0f / 9.0f);
    p = rf_add(rf_mul(p, s2), 1.0f / 7.0f);
    p = rf_add(rf_mul(p, s2), 1.0f / 5.0f);
    p = rf_add(rf_mul(p, s2), 1.0f / 3.0f);
    p = rf_add(rf_mul(p, s2), 1.0f);
    const float ln_m = rf_mul(rf_mul(2.0f, s), p);
    const float ln_u = rf_add(rf_mul((float)(e - 24), 0x1.62e43p-1f), ln_m);
    const float radius = __fsqrt_rn(rf_mul(-2.0f, ln_u));

    // ---- cos(2 pi k2 / 2^24)
    const unsigned int oct = k2 >> 21, r = k2 & 0x1FFFFFu;
    const unsigned int rr = (oct & 1u) ? (0x200000u - r) : r;
    const float x = rf_mul(rf_mul((float)rr, 1.0f / 2097152.0f), 0x1.921fb6p-1f);
    const float x2 = rf_mul(x, x);
    float sn = 1.0f / 362880.0f;
    sn = rf_add(rf_mul(sn, x2), -1.0f / 5040.0f);
    sn = rf_add(rf_mul(sn, x2), 1.0f / 120.0f);
    sn = rf_add(rf_mul(sn, x2), -1.0f / 6.0f);
    sn = rf_add(rf_mul(sn, x2), 1.0f);
    sn = rf_mul(sn, x);
    float cs = -1.0f / 3628800.0f;
    cs = rf_add(rf_mul(cs, x2), 1.0f / 40320.0f);
    cs = rf_add(rf_mul(cs, x2), -1.0f / 720.0f);
    cs = rf_add(rf_mul(cs, x2), 1.0f / 24.0f);
    cs = rf_add(rf_mul(cs, x2), -0.5f);
    cs = rf_add(rf_mul(cs, x2), 1.0f);
    const bool use_sin = oct == 1 || oct == 2 || oct == 5 || oct == 6;
    const bool negative = oct >= 2 && oct <= 5;
    float c = use_sin ? sn : cs;
    if (negative) c = -c;
    return rf_mul(radius, c);
}

template <typename TO>
__global__ void random_fill_kernel(TO* __restrict__ out, size_t n, unsigned long long key, float std, float offset) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(rf_add(offset, rf_mul(rf_normal(key, i), std)));
}

TQ_API int tq_random_fill(void* out, int out_dtype, size_t n, unsigned long long key, float std, float offset,
                          cudaStream_t stream) {
    if (n == 0) return 0;
    const int threads = 256;
    size_t blocks = (n + threads - 1) / threads;
    if (blocks > (size_t)tq_sm_count() * 16) blocks = (size_t)tq_sm_count() * 16;
    if (out_dtype == TQ_F32)
        random_fill_kernel<float><<<(int)blocks, threads, 0, stream>>>((float*)out, n, key, std, offset);
    else if (out_dtype == TQ_BF16)
        random_fill_kernel<bf16><<<(int)blocks, threads, 0, stream>>>((bf16*)out, n, key, std, offset);
    else
        return (int)cudaErrorInvalidValue;
    return tq_launch_status();
}
