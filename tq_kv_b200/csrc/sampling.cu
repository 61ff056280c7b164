// Token selection from float32 logits on the device: arg-max, or
// temperature + top-k + top-p with one uniform draw per row, with an
// optional repeat penalty driven by per-row occurrence counts.
//
// Reference: src/engine.rs:353-360 (temperature <= 0 -> arg-max, else top-k
// then top-p at the temperature), :403-419 (repeat penalty: once per
// occurrence of a generated token, l > 0 ? l / p : l * p).  The sampler proper
// is outside the reference's tree; the rules here are this project's:
//  * arg-max ties go to the lowest token id;
//  * top-k keeps every token whose logit is >= the k-th largest;
//  * top-p walks the kept tokens by descending probability and keeps every
//    token whose probability is >= that of the token at which the running
//    mass first reaches top_p * (kept mass);
//  * the draw walks the kept tokens in token-id order and takes the first
//    one whose running mass exceeds u * (kept mass).
// Probabilities are float32 exponentials, masses are summed in float64.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ float penalised(const float* logits, const int* counts, float penalty, int i) {
    float l = logits[i];
    if (counts) {
        for (int c = counts[i]; c > 0; --c) l = l > 0.f ? l / penalty : l * penalty;
    }
    return l;
}

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// the inverse of order_key
__device__ __forceinline__ float key_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) red[warp] = a;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    ArgMax r = lane < nw ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
        r = better(r, b);
    }
    return r;
}

__device__ double block_sum_f64(double v, double* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum_f64(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    double r = lane < nw ? red[lane] : 0.0;
    return warp_sum_f64(r);
}

// Where a row's uniform draw in [0, 1) comes from: an array the caller filled, or the counter-based generator
// of sampling/rng.py run here: a draw depends on (seed, request index, index of the sampled token) only, so a
// request's output does not depend on what else is in its batch or on the slot it got (the reference seeds one
// generator per call, src/engine.rs:362).  24 random bits, exact in float32.
struct Draws {
    const float* uniforms;           // [rows], or null: generate
    const int* requests;             // [rows] request index of each row
    unsigned long long seed;
    int index;
};
__device__ __forceinline__ unsigned long long draw_mix(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float draw_uniform(const Draws& d, int row) {
    if (d.uniforms) return d.uniforms[row];
    unsigned long long z = draw_mix(d.seed);
    z = draw_mix(z ^ ((unsigned long long)(long long)d.requests[row] * 0xD6E8FEB86659FD93ull));
    z = draw_mix(z ^ ((unsigned long long)(long long)d.index * 0xA0761D6478BD642Full));
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// One block per row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, float temperature, int top_k, float top_p,
              Draws draws, int* __restrict__ counts, float penalty, int* __restrict__ out) {
    __shared__ ArgMax red_am[32];
    __shared__ double red_d[32];
    __shared__ int hist_i[256];
    __shared__ double hist_d[256];
    __shared__ double seg_sum[SAMPLE_THREADS];
    __shared__ uint32_t sh_prefix;
    __shared__ double sh_remaining;
    __shared__ int sh_token;

    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch();
    const float* lg = logits + (size_t)row * ld;
    int* cnt = counts ? counts + (size_t)row * V : nullptr;

    // ---- arg-max (also the softmax's maximum) ----
    ArgMax am{-INFINITY, 0x7fffffff};
    for (int i = tid; i < V; i += blockDim.x) am = better(am, ArgMax{penalised(lg, cnt, penalty, i), i});
    am = block_argmax(am, red_am);
    if (temperature <= 0.f) {
        if (tid == 0) {
            out[row] = am.i;
            if (cnt) cnt[am.i] += 1;
        }
        return;
    }
    const float mx = am.v;

    // ---- top-k: key of the k-th largest logit by radix select ----
    uint32_t kth_key = 0;   // keep everything
    if (top_k > 0 && top_k < V) {
        uint32_t prefix = 0, mask = 0;
        int remaining = top_k;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist_i[tid] = 0;
            __syncthreads();
            for (int i0 = 0; i0 < V; i0 += blockDim.x) {
                const int i = i0 + tid;
                int bin = -1;
                if (i < V) {
                    const uint32_t key = order_key(penalised(lg, cnt, penalty, i));
                    if ((key & mask) == prefix) bin = (key >> shift) & 255;
                }
                // one atomic per distinct bin of the warp
                const unsigned peers = __match_any_sync(0xffffffffu, bin);
                if (bin >= 0 && (tid & 31) == __ffs(peers) - 1) atomicAdd(&hist_i[bin], __popc(peers));
            }
            __syncthreads();
            if (tid == 0) {
                int cum = 0, sel = 0;
                for (int b = 255; b >= 0; --b) {
                    if (cum + hist_i[b] >= remaining) { sel = b; break; }
                    cum += hist_i[b];
                }
                sh_prefix = prefix | ((uint32_t)sel << shift);
                sh_remaining = (double)(remaining - cum);
            }
            __syncthreads();
            prefix = sh_prefix;
            remaining = (int)sh_remaining;
            mask |= 255u << shift;
            __syncthreads();
        }
        kth_key = prefix;
    }

    // ---- top-p: probability bits of the token where the descending mass reaches top_p * kept mass ----
    uint32_t cut_bits = 0;  // keep everything (probabilities are >= 0, their bits order like the values)
    if (top_p < 1.f) {
        double mass = 0.0;
        for (int i = tid; i < V; i += blockDim.x) {
            const float l = penalised(lg, cnt, penalty, i);
            if (order_key(l) >= kth_key) mass += (double)expf((l - mx) / temperature);
        }
        mass = block_sum_f64(mass, red_d);
        uint32_t prefix = 0, mask = 0;
        double remaining = (double)top_p * mass;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hist_d[tid] = 0.0;
            __syncthreads();
            for (int i = tid; i < V; i += blockDim.x) {
                const float l = penalised(lg, cnt, penalty, i);
                if (order_key(l) < kth_key) continue;
                const float p = expf((l - mx) / temperature);
                const uint32_t bits = __float_as_uint(p);
                if ((bits & mask) == prefix) atomicAdd(&hist_d[(bits >> shift) & 255], (double)p);
            }
            __syncthreads();
            if (tid == 0) {
                double cum = 0.0;
                int sel = -1, lowest = 0;
                for (int b = 255; b >= 0; --b) {
                    if (hist_d[b] > 0.0) lowest = b;
                    if (cum + hist_d[b] >= remaining && hist_d[b] > 0.0) { sel = b; break; }
                    cum += hist_d[b];
                }
                if (sel < 0) {                    // rounding left the target just above the total
                    sel = lowest;
                    cum -= hist_d[lowest];
                }
                sh_prefix = prefix | ((uint32_t)sel << shift);
                sh_remaining = remaining - cum;
            }
            __syncthreads();
            prefix = sh_prefix;
            remaining = sh_remaining;
            mask |= 255u << shift;
            __syncthreads();
        }
        cut_bits = prefix;
    }

    // ---- the draw: walk the kept tokens in token-id order ----
    const int seg = (V + blockDim.x - 1) / blockDim.x;
    const int s0 = min(V, tid * seg), s1 = min(V, s0 + seg);
    double mine = 0.0;
    for (int i = s0; i < s1; ++i) {
        const float l = penalised(lg, cnt, penalty, i);
        if (order_key(l) < kth_key) continue;
        const float p = expf((l - mx) / temperature);
        if (__float_as_uint(p) >= cut_bits) mine += (double)p;
    }
    seg_sum[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int t = 0; t < (int)blockDim.x; ++t) total += seg_sum[t];
        const double target = (double)draw_uniform(draws, row) * total;
        double cum = 0.0;
        int owner = -1;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (cum + seg_sum[t] > target && seg_sum[t] > 0.0) { owner = t; break; }
            cum += seg_sum[t];
        }
        if (owner < 0) {                         // rounding: take the last segment that holds mass
            for (int t = (int)blockDim.x - 1; t >= 0; --t)
                if (seg_sum[t] > 0.0) { owner = t; break; }
            cum = -1.0;                           // marks "take the segment's last kept token"
        }
        sh_token = owner;
        sh_remaining = cum;
        red_d[0] = target;
    }
    __syncthreads();
    if (tid == sh_token) {
        const double target = red_d[0];
        double cum = sh_remaining;
        const bool take_last = cum < 0.0;
        int tok = -1, last = -1;
        for (int i = s0; i < s1; ++i) {
            const float l = penalised(lg, cnt, penalty, i);
            if (order_key(l) < kth_key) continue;
            const float p = expf((l - mx) / temperature);
            if (__float_as_uint(p) < cut_bits) continue;
            last = i;
            if (!take_last) {
                cum += (double)p;
                if (cum > target) { tok = i; break; }
            }
        }
        if (tok < 0) tok = last;
        out[row] = tok;
        if (cnt) cnt[tok] += 1;
    }
}


// ---------------------------------------------------------------------------
// Fast path for 0 < top_k <= TOPK_MAX (the usual case: the reference's default
// is 40).  Step 1: every row's vocabulary is cut into TOPK_PARTS parts; a block
// holds its part's keys in shared memory and selects the part's top_k there
// (every token of the row's top k is among its part's top k).  Step 2: one
// block per row selects the row's top k among the candidates and then does
// top-p and the draw on those few tokens with plain sorted sums.  The rules
// are those stated at the top of this file; sums run in the same order as a
// straightforward sorted implementation would run them.
// ---------------------------------------------------------------------------
#define TOPK_MAX 64
#define TOPK_PARTS 32
#define TOPK_CAP 128            // candidates kept per part (top_k plus ties at the cut)
#define TOPK_PART_MAX 8192      // largest part held in shared memory: vocabularies up to 262,144
#define TOPK_KEEP_MAX 512       // tokens kept per row after top-k (top_k plus ties at the cut)

// key of the k-th largest among n keys in shared memory (k <= n); all threads of the block call it
__device__ uint32_t block_kth_largest(const uint32_t* keys, int n, int k, int* hist, uint32_t* sh_prefix,
                                      int* sh_remaining) {
    uint32_t prefix = 0, mask = 0;
    int remaining = k;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const uint32_t key = keys[i];
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int cum = 0, sel = 0;
            for (int b = 255; b >= 0; --b) {
                if (cum + hist[b] >= remaining) { sel = b; break; }
                cum += hist[b];
            }
            *sh_prefix = prefix | ((uint32_t)sel << shift);
            *sh_remaining = remaining - cum;
        }
        __syncthreads();
        prefix = *sh_prefix;
        remaining = *sh_remaining;
        mask |= 255u << shift;
        __syncthreads();
    }
    return prefix;
}

__global__ void __launch_bounds__(256)
topk_parts_kernel(const float* __restrict__ logits, int ld, int V, const int* __restrict__ counts, float penalty,
                  int top_k, float* __restrict__ cand_val, int* __restrict__ cand_idx, int* __restrict__ cand_cnt) {
    __shared__ uint32_t keys[TOPK_PART_MAX];
    __shared__ int hist[256];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_remaining, sh_count;
    const int row = blockIdx.x, part = blockIdx.y;
    pdl_wait();
    pdl_launch();
    const float* lg = logits + (size_t)row * ld;
    const int* cnt = counts ? counts + (size_t)row * V : nullptr;
    const int per = (V + TOPK_PARTS - 1) / TOPK_PARTS;
    const int lo = part * per, n = max(0, min(V, lo + per) - lo);
    for (int i = threadIdx.x; i < n; i += blockDim.x) keys[i] = order_key(penalised(lg, cnt, penalty, lo + i));
    if (threadIdx.x == 0) sh_count = 0;
    __syncthreads();
    uint32_t kth = 0;
    if (n > top_k) kth = block_kth_largest(keys, n, top_k, hist, &sh_prefix, &sh_remaining);
    const size_t base = ((size_t)row * TOPK_PARTS + part) * TOPK_CAP;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (keys[i] >= kth) {
            const int slot = atomicAdd(&sh_count, 1);
            if (slot < TOPK_CAP) {
                cand_val[base + slot] = penalised(lg, cnt, penalty, lo + i);
                cand_idx[base + slot] = lo + i;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) cand_cnt[row * TOPK_PARTS + part] = min(sh_count, TOPK_CAP);
}

__global__ void __launch_bounds__(256)
topk_final_kernel(const float* __restrict__ cand_val, const int* __restrict__ cand_idx,
                  const int* __restrict__ cand_cnt, int V, float temperature, int top_k, float top_p,
                  Draws draws, int* __restrict__ counts, int* __restrict__ out) {
    __shared__ uint32_t keys[TOPK_PARTS * TOPK_CAP];             // order keys of the candidates' logits
    __shared__ int idxs[TOPK_PARTS * TOPK_CAP];
    __shared__ float kp[TOPK_KEEP_MAX], sp[TOPK_KEEP_MAX];       // kept probabilities; the same, sorted
    __shared__ int ki[TOPK_KEEP_MAX], si[TOPK_KEEP_MAX];         // kept token ids; ids in sorted order
    __shared__ int hist[256];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_remaining, sh_n, sh_kept;
    __shared__ float sh_cut;
    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch();
    // gather the candidates of all parts
    if (tid == 0) { sh_n = 0; sh_kept = 0; }
    __syncthreads();
    for (int part = 0; part < TOPK_PARTS; ++part) {
        const int c = cand_cnt[row * TOPK_PARTS + part];
        const size_t base = ((size_t)row * TOPK_PARTS + part) * TOPK_CAP;
        __shared__ int sh_off;
        if (tid == 0) { sh_off = sh_n; sh_n += c; }
        __syncthreads();
        for (int i = tid; i < c; i += blockDim.x) {
            idxs[sh_off + i] = cand_idx[base + i];
            keys[sh_off + i] = order_key(cand_val[base + i]);
        }
        __syncthreads();
    }
    const int n = sh_n;
    uint32_t kth = 0;
    if (n > top_k) kth = block_kth_largest(keys, n, top_k, hist, &sh_prefix, &sh_remaining);
    // the row's maximum and the kept tokens (logit >= the k-th largest)
    float mx = -INFINITY;
    for (int i = tid; i < n; i += blockDim.x) mx = fmaxf(mx, key_value(keys[i]));
    __shared__ float red[32];
    mx = block_max(mx, red);
    for (int i = tid; i < n; i += blockDim.x) {
        if (keys[i] >= kth) {
            const int slot = atomicAdd(&sh_kept, 1);
            if (slot < TOPK_KEEP_MAX) {
                kp[slot] = expf((key_value(keys[i]) - mx) / temperature);
                ki[slot] = idxs[i];
            }
        }
    }
    __syncthreads();
    const int m = min(sh_kept, TOPK_KEEP_MAX);
    // top-p: sort by probability (descending, lower id first on ties), running mass in float64
    for (int e = tid; e < m; e += blockDim.x) {
        int rank = 0;
        for (int j = 0; j < m; ++j) rank += (kp[j] > kp[e] || (kp[j] == kp[e] && ki[j] < ki[e])) ? 1 : 0;
        sp[rank] = kp[e];
    }
    __syncthreads();
    if (tid == 0) {
        float cut = 0.f;
        if (top_p < 1.f) {
            double total = 0.0;
            for (int j = 0; j < m; ++j) total += (double)sp[j];
            const double target = (double)top_p * total;
            double cum = 0.0;
            cut = sp[m - 1];
            for (int j = 0; j < m; ++j) {
                cum += (double)sp[j];
                if (cum >= target) { cut = sp[j]; break; }
            }
        }
        sh_cut = cut;
    }
    __syncthreads();
    const float cut = sh_cut;
    // the draw: kept tokens in token-id order
    for (int e = tid; e < m; e += blockDim.x) {
        int rank = 0;
        for (int j = 0; j < m; ++j) rank += (ki[j] < ki[e]) ? 1 : 0;
        si[rank] = ki[e];
        sp[rank] = kp[e] >= cut ? kp[e] : 0.f;
    }
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int j = 0; j < m; ++j) total += (double)sp[j];
        const double target = (double)draw_uniform(draws, row) * total;
        double cum = 0.0;
        int tok = -1, last = -1;
        for (int j = 0; j < m; ++j) {
            if (sp[j] > 0.f) last = si[j];
            cum += (double)sp[j];
            if (cum > target) { tok = si[j]; break; }
        }
        if (tok < 0) tok = last;
        out[row] = tok;
        if (counts) counts[(size_t)row * V + tok] += 1;
    }
}

// Arg-max in two steps for speed: the vocabulary of a row is cut into ARGMAX_PARTS parts, one block each;
// a second kernel picks the best part (lowest id on ties) and counts the chosen token.
#define ARGMAX_PARTS 32

__global__ void __launch_bounds__(256)
argmax_parts_kernel(const float* __restrict__ logits, int ld, int V, const int* __restrict__ counts, float penalty,
                    ArgMax* __restrict__ parts) {
    __shared__ ArgMax red[32];
    const int row = blockIdx.x, part = blockIdx.y;
    pdl_wait();
    pdl_launch();
    const float* lg = logits + (size_t)row * ld;
    const int* cnt = counts ? counts + (size_t)row * V : nullptr;
    const int per = (V + ARGMAX_PARTS - 1) / ARGMAX_PARTS;
    const int lo = part * per, hi = min(V, lo + per);
    ArgMax am{-INFINITY, 0x7fffffff};
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) am = better(am, ArgMax{penalised(lg, cnt, penalty, i), i});
    am = block_argmax(am, red);
    if (threadIdx.x == 0) parts[row * ARGMAX_PARTS + part] = am;
}

__global__ void argmax_final_kernel(const ArgMax* __restrict__ parts, int* __restrict__ counts, int V,
                                    int* __restrict__ out) {
    const int row = blockIdx.x, lane = threadIdx.x;
    pdl_wait();
    pdl_launch();
    ArgMax a = lane < ARGMAX_PARTS ? parts[row * ARGMAX_PARTS + lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
        a = better(a, b);
    }
    if (lane == 0) {
        out[row] = a.i;
        if (counts) counts[(size_t)row * V + a.i] += 1;
    }
}

// counts: int32 [rows, V] occurrence counts of generated tokens (or null);
// the sampled token's count is incremented.  uniforms: float [rows] in [0, 1)
// (unused when temperature <= 0).
// scratch: optional, tq_sample_scratch_bytes(rows) bytes; with it, arg-max and sampling with
// 0 < top_k <= 64 run as two short kernels on many blocks instead of one block per row.
TQ_API size_t tq_sample_scratch_bytes(int n_rows) {
    return (size_t)n_rows * TOPK_PARTS * (TOPK_CAP * 8 + 4) + 256;
}

static int sample_launch(const float* logits, int ld, int n_rows, int V, float temperature, int top_k, float top_p,
                         Draws draws, int* counts, float penalty, int* out, void* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (V <= 0 || ld < V) return (int)cudaErrorInvalidValue;
    if (temperature > 0.f && !draws.uniforms && !draws.requests) return (int)cudaErrorInvalidValue;
    if (counts && !(penalty > 0.f)) return (int)cudaErrorInvalidValue;
    if (temperature <= 0.f && scratch && n_rows <= 65535) {
        int st = tq_launch_pdl(TQ_PDL_SAMPLING, argmax_parts_kernel, dim3(n_rows, ARGMAX_PARTS), dim3(256), 0, stream, logits, ld, V,
                               (const int*)counts, penalty, (ArgMax*)scratch);
        if (st) return st;
        return tq_launch_pdl(TQ_PDL_SAMPLING, argmax_final_kernel, dim3(n_rows), dim3(32), 0, stream, (const ArgMax*)scratch, counts, V,
                             out);
    }
    if (temperature > 0.f && scratch && top_k > 0 && top_k <= TOPK_MAX && n_rows <= 65535 &&
        (V + TOPK_PARTS - 1) / TOPK_PARTS <= TOPK_PART_MAX) {
        float* cand_val = (float*)scratch;
        int* cand_idx = (int*)(cand_val + (size_t)n_rows * TOPK_PARTS * TOPK_CAP);
        int* cand_cnt = cand_idx + (size_t)n_rows * TOPK_PARTS * TOPK_CAP;
        int st = tq_launch_pdl(TQ_PDL_SAMPLING, topk_parts_kernel, dim3(n_rows, TOPK_PARTS), dim3(256), 0, stream, logits, ld, V,
                               (const int*)counts, penalty, top_k, cand_val, cand_idx, cand_cnt);
        if (st) return st;
        return tq_launch_pdl(TQ_PDL_SAMPLING, topk_final_kernel, dim3(n_rows), dim3(256), 0, stream, (const float*)cand_val,
                             (const int*)cand_idx, (const int*)cand_cnt, V, temperature, top_k, top_p, draws,
                             counts, out);
    }
    return tq_launch_pdl(TQ_PDL_SAMPLING, sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, ld, V, temperature,
                         top_k, top_p, draws, counts, penalty, out);
}

TQ_API int tq_sample(const float* logits, int ld, int n_rows, int V, float temperature, int top_k, float top_p,
                     const float* uniforms, int* counts, float penalty, int* out, void* scratch,
                     cudaStream_t stream) {
    return sample_launch(logits, ld, n_rows, V, temperature, top_k, top_p, Draws{uniforms, nullptr, 0ull, 0}, counts,
                         penalty, out, scratch, stream);
}

// The same with the rows' draws generated on the device: requests [rows] int32 (the request index of each row),
// the generation's seed and the index of the token being sampled (see Draws).
TQ_API int tq_sample_seeded(const float* logits, int ld, int n_rows, int V, float temperature, int top_k, float top_p,
                            const int* requests, unsigned long long seed, int index, int* counts, float penalty,
                            int* out, void* scratch, cudaStream_t stream) {
    return sample_launch(logits, ld, n_rows, V, temperature, top_k, top_p, Draws{nullptr, requests, seed, index}, counts,
                         penalty, out, scratch, stream);
}
