// Memory-bound kernels around the matrix products: embedding gather, RMS
// norm, bias + rotary position encoding + cache append, SwiGLU gating.
// All arithmetic is float32; T* parameters are float or bfloat16.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = float(table[tokens[t], :])
// (src/models/turbo_generic.rs:1958 — a row gather, no scaling.)
// A token id outside [0, V) writes zeros and raises bit 0 of *status.
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                             float* __restrict__ out, int H, int V, int* status) {
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const int id = tokens[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        return;
    }
    const TW* row = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32<TW>(row[i]);
}

TQ_API int tq_embed(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens, int H, int V,
                    int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                             (const float*)table, out, H, V, status);
    if (table_dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                             (const bf16*)table, out, H, V, status);
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// RMS norm: y = x / sqrt(mean(x^2) + eps) * w, all in float32
// (src/models/turbo_generic.rs:41-51).  x is the float32 residual stream;
// `rows` (optional) selects the input rows, so that the final norm touches
// only the rows whose logits are wanted.
// ---------------------------------------------------------------------------
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    TO* o = out + (size_t)r * H;
    float ss = 0.f;
    if ((H & 3) == 0) {                       // rows are 16-byte aligned: four values per load
        const float4* x4 = reinterpret_cast<const float4*>(xr);
        const float4* w4 = reinterpret_cast<const float4*>(w);
        for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
            const float4 v = x4[i];
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
        ss = block_sum(ss, red);
        const float rms = sqrtf(ss / (float)H + eps);
        for (int i = threadIdx.x; i < (H >> 2); i += blockDim.x) {
            const float4 v = x4[i], g = w4[i];
            store2_f32<TO>(o + 4 * i, (v.x / rms) * g.x, (v.y / rms) * g.y);
            store2_f32<TO>(o + 4 * i + 2, (v.z / rms) * g.z, (v.w / rms) * g.w);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<TO>((xr[i] / rms) * w[i]);
}

// Rows of up to 8,192 values in steps of four: a row is read once and held in registers between the sum of
// squares and the scaling (VPT 16-byte loads per thread, all in flight together, the norm's weights with them).
// A prompt's many rows get small blocks, so that a whole wave of rows is resident; the few rows of a decode
// step get wide ones, so that a row is one round of loads.  Same arithmetic as above.
template <typename TO, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_cached_kernel(const float* __restrict__ x, const float* __restrict__ w, TO* __restrict__ out,
                      const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x, h4 = H >> 2;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    TO* o = out + (size_t)r * H;
    float4 v[VPT], g[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {                        // the weights do not depend on the kernel before
        const int idx = threadIdx.x + i * THREADS;
        g[i] = idx < h4 ? w4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    pdl_launch();
    const float4* x4 = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        v[i] = idx < h4 ? x4[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < h4) {
            store2_f32<TO>(o + 4 * idx, (v[i].x / rms) * g[i].x, (v[i].y / rms) * g[i].y);
            store2_f32<TO>(o + 4 * idx + 2, (v[i].z / rms) * g[i].z, (v[i].w / rms) * g[i].w);
        }
    }
}

template <typename TO>
static int launch_rmsnorm_cached(const float* x, const float* w, TO* out, const int* rows, int n_rows, int H, float eps,
                                 cudaStream_t stream) {
    const int h4 = H >> 2;
#define TQ_RN(T, V)                                                                                                 \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, rmsnorm_cached_kernel<TO, T, V>, dim3(n_rows), dim3(T), 0, stream, x, w, \
                         out, rows, H, eps)
    if (n_rows < 128) {                                    // a decode step: wide blocks
        if (h4 <= 128) TQ_RN(128, 1);
        if (h4 <= 512) TQ_RN(512, 1);
        if (h4 <= 1024) TQ_RN(512, 2);
        TQ_RN(512, 4);
    }
    if (h4 <= 128 * 2) TQ_RN(128, 2);
    if (h4 <= 128 * 4) TQ_RN(128, 4);
    if (h4 <= 128 * 8) TQ_RN(128, 8);
    TQ_RN(256, 8);
#undef TQ_RN
}

TQ_API int tq_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows, int H,
                      float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((H & 3) == 0 && H <= 256 * 8 * 4 && (out_dtype == TQ_F32 || out_dtype == TQ_BF16)) {
        if (out_dtype == TQ_F32) return launch_rmsnorm_cached<float>(x, w, (float*)out, rows, n_rows, H, eps, stream);
        return launch_rmsnorm_cached<bf16>(x, w, (bf16*)out, rows, n_rows, H, eps, stream);
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (out_dtype == TQ_F32)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, (float*)out, rows,
                             H, eps);
    if (out_dtype == TQ_BF16)
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, w, (bf16*)out, rows, H,
                             eps);
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// Bias + rotate-half rotary encoding + head split + cache append.
//
// qkv: [T, (nh + 2*nkv) * hd] — q heads, then k heads, then v heads, each
// head-major (src/models/turbo_generic.rs:815-817).  Bias is added first
// (:805-813), then q and k are rotated (:417-427):
//   out[:half] = x0*cos - x1*sin, out[half:] = x0*sin + x1*cos
// over the first `rot` dims of a head (half = rot/2), with cos/sin rows taken
// at the token's absolute position from tables [positions, rot/2] (:746-768).
// q goes to q_out [T, nh*hd]; k and v go to the packed outputs (if given)
// and into the paged cache (if given): position p of step row b lands in
// logical page p / page_tokens (modulo ring_pages if > 0) at row
// p % page_tokens.  In a ring, only the last ring_pages*page_tokens positions
// of a sequence are written, so that no two tokens of one step meet in a row.
// A row whose position is not below new_lens of its sequence is padding (a
// prompt padded to the size of a captured graph): it gets q (and packed k, v)
// like any row and leaves the cache alone.
// ---------------------------------------------------------------------------
template <typename TI, typename TC>
__global__ void qkv_rope_cache_kernel(const TI* __restrict__ qkv, const float* __restrict__ bias,
                                      const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                      const int* __restrict__ new_lens, const int* __restrict__ block_table,
                                      int table_width, int ring_pages, int page_tokens, TC* __restrict__ q_out,
                                      TC* __restrict__ k_out, TC* __restrict__ v_out, TC* __restrict__ k_pages,
                                      TC* __restrict__ v_pages, int nh, int nkv, int hd, int rot, int clear_in) {
    // grid (token, head): heads 0..nh-1 are q, nh..nh+nkv-1 are k, the rest are v
    // The step's positions and tables were copied in before its first kernel ran: only qkv depends on the
    // kernel before, so the addressing is done before waiting for it.
    const int t = blockIdx.x, head = blockIdx.y;
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const int half = rot >> 1;
    const int width = (nh + 2 * nkv) * hd;
    const TI* x = qkv + (size_t)t * width + (size_t)head * hd;
    const float* bs = bias ? bias + (size_t)head * hd : nullptr;
    const bool is_q = head < nh, is_k = !is_q && head < nh + nkv;
    const int g = is_q ? 0 : (is_k ? head - nh : head - nh - nkv);

    // where this token's key/value row lives in the cache (or nowhere)
    TC* cache = nullptr;
    if (!is_q && k_pages != nullptr) {
        int lp = pos / page_tokens;
        bool keep = pos < new_lens[b];          // a row past its sequence's new length is padding: nothing is cached
        if (ring_pages > 0) {
            keep = keep && pos >= new_lens[b] - ring_pages * page_tokens;
            lp %= ring_pages;
        }
        if (keep) {
            const int page = block_table[(size_t)b * table_width + lp];
            const size_t row = (((size_t)page * nkv + g) * page_tokens + (pos % page_tokens)) * hd;
            cache = (is_k ? k_pages : v_pages) + row;
        }
    }
    TC* dst = is_q ? q_out + ((size_t)t * nh + head) * hd
                   : (is_k ? (k_out ? k_out + ((size_t)t * nkv + g) * hd : nullptr)
                           : (v_out ? v_out + ((size_t)t * nkv + g) * hd : nullptr));
    pdl_wait();
    pdl_launch();
    if (is_q || is_k) {
        const float* cs = cos_tab + (size_t)pos * half;
        const float* sn = sin_tab + (size_t)pos * half;
        for (int j = threadIdx.x; j < half; j += blockDim.x) {
            float x0 = to_f32<TI>(x[j]), x1 = to_f32<TI>(x[j + half]);
            if (bs) { x0 += bs[j]; x1 += bs[j + half]; }
            const float c = cs[j], s = sn[j];
            const TC r0 = from_f32<TC>(x0 * c - x1 * s);
            const TC r1 = from_f32<TC>(x0 * s + x1 * c);
            if (dst) { dst[j] = r0; dst[j + half] = r1; }
            if (cache) { cache[j] = r0; cache[j + half] = r1; }
        }
        for (int d = rot + threadIdx.x; d < hd; d += blockDim.x) {      // dims beyond the rotated part pass through
            float v = to_f32<TI>(x[d]);
            if (bs) v += bs[d];
            const TC r = from_f32<TC>(v);
            if (dst) dst[d] = r;
            if (cache) cache[d] = r;
        }
    } else {
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {             // values: bias only
            float v = to_f32<TI>(x[d]);
            if (bs) v += bs[d];
            const TC r = from_f32<TC>(v);
            if (dst) dst[d] = r;
            if (cache) cache[d] = r;
        }
    }
    // clear_in: this block alone has read its head's slice of qkv and leaves zeros there, so that the next
    // product that adds its shares of K into the same buffer needs no clearing of its own
    if (clear_in) {
        __syncthreads();
        TI* xz = const_cast<TI*>(x);
        for (int d = threadIdx.x; d < hd; d += blockDim.x) xz[d] = from_f32<TI>(0.f);
    }
}

// The same for the common serving case (float32 in, bfloat16 out, the whole head rotated, head_dim a
// multiple of 8): one block per token, every thread handles four neighbouring dims with 16-byte loads.
__device__ __forceinline__ uint2 pack4_bf16(float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    return make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

__global__ void __launch_bounds__(256)
qkv_rope_cache_vec_kernel(const float* __restrict__ qkv, const float* __restrict__ bias,
                          const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                          const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                          const int* __restrict__ new_lens, const int* __restrict__ block_table, int table_width,
                          int ring_pages, int page_tokens, bf16* __restrict__ q_out, bf16* __restrict__ k_out,
                          bf16* __restrict__ v_out, bf16* __restrict__ k_pages, bf16* __restrict__ v_pages, int nh,
                          int nkv, int hd) {
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const int pos = tok_pos[t];
    const int b = tok_seq[t];
    const int half = hd >> 1, q4 = half >> 2;
    const float* x = qkv + (size_t)t * (nh + 2 * nkv) * hd;
    const float* cs = cos_tab + (size_t)pos * half;
    const float* sn = sin_tab + (size_t)pos * half;
    size_t cache_row = 0;
    bool to_cache = k_pages != nullptr && pos < new_lens[b];       // (rows past the new length are padding)
    if (to_cache) {
        int lp = pos / page_tokens;
        if (ring_pages > 0) {
            if (pos < new_lens[b] - ring_pages * page_tokens) to_cache = false;
            lp %= ring_pages;
        }
        if (to_cache)
            cache_row = ((size_t)block_table[(size_t)b * table_width + lp] * nkv) * page_tokens + (pos % page_tokens);
    }
    for (int idx = threadIdx.x; idx < (nh + nkv) * q4; idx += blockDim.x) {
        const int head = idx / q4, j = (idx - head * q4) * 4;
        const int c0 = head * hd + j;
        float4 x0 = *reinterpret_cast<const float4*>(x + c0);
        float4 x1 = *reinterpret_cast<const float4*>(x + c0 + half);
        if (bias) {
            const float4 b0 = *reinterpret_cast<const float4*>(bias + c0);
            const float4 b1 = *reinterpret_cast<const float4*>(bias + c0 + half);
            x0.x += b0.x; x0.y += b0.y; x0.z += b0.z; x0.w += b0.w;
            x1.x += b1.x; x1.y += b1.y; x1.z += b1.z; x1.w += b1.w;
        }
        const float4 c = *reinterpret_cast<const float4*>(cs + j);
        const float4 s = *reinterpret_cast<const float4*>(sn + j);
        const uint2 r0 = pack4_bf16(x0.x * c.x - x1.x * s.x, x0.y * c.y - x1.y * s.y, x0.z * c.z - x1.z * s.z,
                                    x0.w * c.w - x1.w * s.w);
        const uint2 r1 = pack4_bf16(x0.x * s.x + x1.x * c.x, x0.y * s.y + x1.y * c.y, x0.z * s.z + x1.z * c.z,
                                    x0.w * s.w + x1.w * c.w);
        if (head < nh) {
            bf16* q = q_out + ((size_t)t * nh + head) * hd + j;
            *reinterpret_cast<uint2*>(q) = r0;
            *reinterpret_cast<uint2*>(q + half) = r1;
        } else {
            const int g = head - nh;
            if (k_out) {
                bf16* k = k_out + ((size_t)t * nkv + g) * hd + j;
                *reinterpret_cast<uint2*>(k) = r0;
                *reinterpret_cast<uint2*>(k + half) = r1;
            }
            if (to_cache) {
                bf16* k = k_pages + (cache_row + (size_t)g * page_tokens) * hd + j;
                *reinterpret_cast<uint2*>(k) = r0;
                *reinterpret_cast<uint2*>(k + half) = r1;
            }
        }
    }
    const int v0 = (nh + nkv) * hd;
    for (int idx = threadIdx.x; idx < nkv * (hd >> 2); idx += blockDim.x) {
        const int g = idx / (hd >> 2), d = (idx - g * (hd >> 2)) * 4;
        float4 v = *reinterpret_cast<const float4*>(x + v0 + g * hd + d);
        if (bias) {
            const float4 bv = *reinterpret_cast<const float4*>(bias + v0 + g * hd + d);
            v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
        }
        const uint2 r = pack4_bf16(v.x, v.y, v.z, v.w);
        if (v_out) *reinterpret_cast<uint2*>(v_out + ((size_t)t * nkv + g) * hd + d) = r;
        if (to_cache) *reinterpret_cast<uint2*>(v_pages + (cache_row + (size_t)g * page_tokens) * hd + d) = r;
    }
}

TQ_API int tq_qkv_rope_cache(const void* qkv, int in_dtype, const float* bias, const float* cos_tab,
                             const float* sin_tab, const int* tok_pos, const int* tok_seq, const int* new_lens,
                             const int* block_table, int table_width, int ring_pages, int page_tokens, void* q_out,
                             void* k_out, void* v_out, void* k_pages, void* v_pages, int cache_dtype, int n_tokens,
                             int nh, int nkv, int hd, int rot, int clear_in, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot <= 0 || rot > hd || (rot & 1) || page_tokens <= 0) return (int)cudaErrorInvalidValue;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return (int)cudaErrorInvalidValue;
    if (k_pages && !block_table) return (int)cudaErrorInvalidValue;
    if (nh + 2 * nkv > 65535) return (int)cudaErrorInvalidValue;
    // many tokens: one block per token with 16-byte accesses; few tokens (decoding): one block per (token, head)
    if (!clear_in && n_tokens >= 128 && in_dtype == TQ_F32 && cache_dtype == TQ_BF16 && rot == hd && (hd & 7) == 0 &&
        (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 && (!bias || (reinterpret_cast<uintptr_t>(bias) & 15) == 0))
        return tq_launch_pdl(TQ_PDL_ELEMENTWISE, qkv_rope_cache_vec_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)qkv,
                             bias, cos_tab, sin_tab, tok_pos, tok_seq, new_lens, block_table, table_width,
                             ring_pages, page_tokens, (bf16*)q_out, (bf16*)k_out, (bf16*)v_out, (bf16*)k_pages,
                             (bf16*)v_pages, nh, nkv, hd);
    const int threads = hd >= 128 ? 64 : 32;
    const dim3 grid(n_tokens, nh + 2 * nkv);
#define TQ_LAUNCH(TI, TC)                                                                                       \
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, qkv_rope_cache_kernel<TI, TC>, grid, dim3(threads), 0, stream, (const TI*)qkv, bias,  \
                         cos_tab, sin_tab, tok_pos, tok_seq, new_lens, block_table, table_width, ring_pages,   \
                         page_tokens, (TC*)q_out, (TC*)k_out, (TC*)v_out, (TC*)k_pages, (TC*)v_pages, nh, nkv, \
                         hd, rot, clear_in)
    if (in_dtype == TQ_F32 && cache_dtype == TQ_F32) TQ_LAUNCH(float, float);
    if (in_dtype == TQ_F32 && cache_dtype == TQ_BF16) TQ_LAUNCH(float, bf16);
    if (in_dtype == TQ_BF16 && cache_dtype == TQ_BF16) TQ_LAUNCH(bf16, bf16);
#undef TQ_LAUNCH
    return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// SwiGLU gating: out[t, i] = silu(gu[t, i]) * gu[t, I + i], silu(x) = x * sigmoid(x)
// (src/models/turbo_generic.rs:105-110, :64-66).  gu holds the gate columns
// first, then the up columns.
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int I, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_f32<TI>(gu[t * 2 * I + i]);
        const float u = to_f32<TI>(gu[t * 2 * I + I + i]);
        const float s = g / (1.f + expf(-g));
        out[idx] = from_f32<TO>(s * u);
    }
}

TQ_API int tq_swiglu(const void* gu, int in_dtype, void* out, int out_dtype, int n_rows, int I, cudaStream_t stream) {
    const size_t total = (size_t)n_rows * I;
    if (total == 0) return 0;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > (size_t)tq_sm_count() * 32) blocks = (size_t)tq_sm_count() * 32;
#define TQ_LAUNCH(TI, TO) \
    swiglu_kernel<TI, TO><<<(int)blocks, threads, 0, stream>>>((const TI*)gu, (TO*)out, I, total)
    if (in_dtype == TQ_F32 && out_dtype == TQ_F32) TQ_LAUNCH(float, float);
    else if (in_dtype == TQ_F32 && out_dtype == TQ_BF16) TQ_LAUNCH(float, bf16);
    else if (in_dtype == TQ_BF16 && out_dtype == TQ_BF16) TQ_LAUNCH(bf16, bf16);
    else return (int)cudaErrorInvalidValue;
#undef TQ_LAUNCH
    return tq_launch_status();
}

// ---------------------------------------------------------------------------
// acc[i] += float(x[i]) — the residual sum in float32 when a library matrix
// product produced the addend.
// ---------------------------------------------------------------------------
template <typename TI>
__global__ void add_into_kernel(float* __restrict__ acc, const TI* __restrict__ x, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        acc[idx] += to_f32<TI>(x[idx]);
}

TQ_API int tq_add_into(float* acc, const void* x, int in_dtype, size_t total, cudaStream_t stream) {
    if (total == 0) return 0;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > (size_t)tq_sm_count() * 32) blocks = (size_t)tq_sm_count() * 32;
    if (in_dtype == TQ_F32) add_into_kernel<float><<<(int)blocks, threads, 0, stream>>>(acc, (const float*)x, total);
    else if (in_dtype == TQ_BF16) add_into_kernel<bf16><<<(int)blocks, threads, 0, stream>>>(acc, (const bf16*)x, total);
    else return (int)cudaErrorInvalidValue;
    return tq_launch_status();
}

// ---------------------------------------------------------------------------
// tokens[i] = sampled[src[i]] where src[i] >= 0: the next token of a sequence
// taken from the sampler's output on the device (row src[i] of the ids it
// wrote last), so that decode steps can follow one another without the host
// reading a token back in between.  Entries with src[i] < 0 keep the id the
// host put there.
// ---------------------------------------------------------------------------
__global__ void select_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src,
                                     const int* __restrict__ sampled, int n) {
    pdl_wait();
    pdl_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int s = src[i];
        if (s >= 0) tokens[i] = sampled[s];
    }
}

TQ_API int tq_select_tokens(int* tokens, const int* src, const int* sampled, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    return tq_launch_pdl(TQ_PDL_ELEMENTWISE, select_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens,
                         src, sampled, n);
}
