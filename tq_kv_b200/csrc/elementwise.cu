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
        return tq_launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
                             (const float*)table, out, H, V, status);
    if (table_dtype == TQ_BF16)
        return tq_launch_pdl(embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, tokens,
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

TQ_API int tq_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows, int n_rows, int H,
                      float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (out_dtype == TQ_F32)
        return tq_launch_pdl(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, w, (float*)out, rows,
                             H, eps);
    if (out_dtype == TQ_BF16)
        return tq_launch_pdl(rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, x, w, (bf16*)out, rows, H,
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
// ---------------------------------------------------------------------------
template <typename TI, typename TC>
__global__ void qkv_rope_cache_kernel(const TI* __restrict__ qkv, const float* __restrict__ bias,
                                      const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                      const int* __restrict__ new_lens, const int* __restrict__ block_table,
                                      int table_width, int ring_pages, int page_tokens, TC* __restrict__ q_out,
                                      TC* __restrict__ k_out, TC* __restrict__ v_out, TC* __restrict__ k_pages,
                                      TC* __restrict__ v_pages, int nh, int nkv, int hd, int rot) {
    // grid (token, head): heads 0..nh-1 are q, nh..nh+nkv-1 are k, the rest are v
    const int t = blockIdx.x, head = blockIdx.y;
    pdl_wait();
    pdl_launch();
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
        bool keep = true;
        if (ring_pages > 0) {
            keep = pos >= new_lens[b] - ring_pages * page_tokens;
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
}

TQ_API int tq_qkv_rope_cache(const void* qkv, int in_dtype, const float* bias, const float* cos_tab,
                             const float* sin_tab, const int* tok_pos, const int* tok_seq, const int* new_lens,
                             const int* block_table, int table_width, int ring_pages, int page_tokens, void* q_out,
                             void* k_out, void* v_out, void* k_pages, void* v_pages, int cache_dtype, int n_tokens,
                             int nh, int nkv, int hd, int rot, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot <= 0 || rot > hd || (rot & 1) || page_tokens <= 0) return (int)cudaErrorInvalidValue;
    if ((k_pages == nullptr) != (v_pages == nullptr)) return (int)cudaErrorInvalidValue;
    if (k_pages && !block_table) return (int)cudaErrorInvalidValue;
    if (nh + 2 * nkv > 65535) return (int)cudaErrorInvalidValue;
    const int threads = hd >= 128 ? 64 : 32;
    const dim3 grid(n_tokens, nh + 2 * nkv);
#define TQ_LAUNCH(TI, TC)                                                                                       \
    return tq_launch_pdl(qkv_rope_cache_kernel<TI, TC>, grid, dim3(threads), 0, stream, (const TI*)qkv, bias,  \
                         cos_tab, sin_tab, tok_pos, tok_seq, new_lens, block_table, table_width, ring_pages,   \
                         page_tokens, (TC*)q_out, (TC*)k_out, (TC*)v_out, (TC*)k_pages, (TC*)v_pages, nh, nkv, \
                         hd, rot)
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
    if (blocks > 148 * 32) blocks = 148 * 32;
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
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (in_dtype == TQ_F32) add_into_kernel<float><<<(int)blocks, threads, 0, stream>>>(acc, (const float*)x, total);
    else if (in_dtype == TQ_BF16) add_into_kernel<bf16><<<(int)blocks, threads, 0, stream>>>(acc, (const bf16*)x, total);
    else return (int)cudaErrorInvalidValue;
    return tq_launch_status();
}
