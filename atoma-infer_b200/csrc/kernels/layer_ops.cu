// Kernels of layers that are not the plain pre-norm block: a short causal convolution over time with its state,
// the norm that comes after the sum, the preparation of attention rows whose queries and keys are normalised as
// whole projections (with biases, a partial rotation and a mix of an earlier layer's values), and the polynomial
// activation of normalised powers.  float32 and bfloat16 storage alike; all arithmetic is float32, and every
// reduction runs in an order that depends only on the row it belongs to.
#include "common.cuh"

// ----------------------------------------------------------------------------- short convolution over time
// What a sublayer reads: y[t] = x[t] * (1 or 0) + sum_j w[c, j] * x[t - taps + 1 + j], x the float32 residual
// stream, zeros before the start of a request.  Rows before the step's portion come from the request's state: a
// ring of R = taps - 1 rows per state slot (slot_stride floats from one slot to the next), the row of position p at
// ring place p mod R.  The state is written by
// short_conv_save (or by the norm kernel below) AFTER this kernel has read it: only the last R rows of an entry
// are written, and within a step they land on places whose old rows this kernel may still need.
template <typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ state,
                  TO* __restrict__ y, const int* __restrict__ meta, const int* __restrict__ positions,
                  const int* __restrict__ token_entry, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, int C, int taps, int add_input, long long slot_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int e = token_entry[t], p = positions[t], first = cu_tokens[e], R = taps - 1;
    const float* st = state + (size_t)slots[e] * slot_stride;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float* wc = w + (size_t)c * taps;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {  // oldest tap first: a fixed order
            const int back = taps - 1 - j, src = p - back;
            if (src < 0) continue;
            const float v = (t - back >= first) ? x[(size_t)(t - back) * C + c] : st[(size_t)(src % R) * C + c];
            acc = fmaf(wc[j], v, acc);
        }
        if (add_input) acc += x[(size_t)t * C + c];
        y[(size_t)t * C + c] = from_float<TO>(acc);
    }
}

extern "C" int short_conv(const float* x, const float* w, const float* state, void* y, int y_dtype, const int* meta,
                          const int* positions, const int* token_entry, const int* cu_tokens, const int* slots, int T,
                          int C, int taps, int add_input, long long slot_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = C >= 1024 ? 256 : 128;
    if (y_dtype == DT_F32)
        return (int)launch_kernel(short_conv_kernel<float>, T, threads, 0, stream, x, w, state, (float*)y, meta, positions,
                                  token_entry, cu_tokens, slots, C, taps, add_input, slot_stride);
    return (int)launch_kernel(short_conv_kernel<__nv_bfloat16>, T, threads, 0, stream, x, w, state, (__nv_bfloat16*)y, meta,
                              positions, token_entry, cu_tokens, slots, C, taps, add_input, slot_stride);
}

// Whether row t is one of the last R rows of its entry, i.e. one the state keeps.
__device__ __forceinline__ bool keeps_row(int t, int e, const int* __restrict__ cu_tokens, int R) {
    return t >= cu_tokens[e + 1] - R;
}

__global__ void __launch_bounds__(256)
short_conv_save_kernel(const float* __restrict__ x, float* __restrict__ state, const int* __restrict__ meta,
                       const int* __restrict__ positions, const int* __restrict__ token_entry,
                       const int* __restrict__ cu_tokens, const int* __restrict__ slots, int C, int R, long long slot_stride) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int e = token_entry[t];
    if (!keeps_row(t, e, cu_tokens, R)) return;
    float* st = state + (size_t)slots[e] * slot_stride + (size_t)(positions[t] % R) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) st[c] = x[(size_t)t * C + c];
}

extern "C" int short_conv_save(const float* x, float* state, const int* meta, const int* positions, const int* token_entry,
                               const int* cu_tokens, const int* slots, int T, int C, int taps, long long slot_stride,
                               cudaStream_t stream) {
    if (T <= 0 || taps <= 1) return 0;
    return (int)launch_kernel(short_conv_save_kernel, T, C >= 1024 ? 256 : 128, 0, stream, x, state, meta, positions,
                              token_entry, cu_tokens, slots, C, taps - 1, slot_stride);
}

// ----------------------------------------------------------------------------- norm after the sum
// resid[t] <- (alpha * resid[t] + delta[t]) * rsqrt(mean(.^2) + eps) * w, the float32 residual stream updated
// in place.  Optional, fused:
//  * keep (a ring as above): the row as it was BEFORE the update is what the sublayer of this sum read; the last
//    rows of every entry go to the state of that sublayer's convolution;
//  * conv_w / conv_state / conv_out: the sublayer after this norm reads the new rows through its own short
//    convolution; for decode steps (every entry one row, so every earlier row comes from the state) this kernel
//    also leaves that sublayer's input, new row + conv(new row, state), in conv_out.
template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
scaled_add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, float alpha, const float* __restrict__ w,
                          float eps, const int* __restrict__ meta, int H, float* __restrict__ keep, int keep_rows,
                          long long keep_stride, long long conv_stride,
                          const int* __restrict__ positions, const int* __restrict__ token_entry,
                          const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                          const float* __restrict__ conv_w, const float* __restrict__ conv_state, int conv_taps,
                          TO* __restrict__ conv_out) {
    __shared__ float red[33];
    extern __shared__ float row[];  // H floats
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    float* x = resid + (size_t)t * H;
    const TD* dl = delta ? delta + (size_t)t * H : nullptr;
    const int e = (keep || conv_out) ? token_entry[t] : 0;
    float* kept = nullptr;
    if (keep && keeps_row(t, e, cu_tokens, keep_rows))
        kept = keep + (size_t)slots[e] * keep_stride + (size_t)(positions[t] % keep_rows) * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float old = x[i];
        if (kept) kept[i] = old;
        const float v = dl ? fmaf(alpha, old, to_float(dl[i])) : alpha * old;
        row[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    const int R = conv_taps - 1;
    const int p = conv_out ? positions[t] : 0;
    const float* st = conv_out ? conv_state + (size_t)slots[e] * conv_stride : nullptr;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row[i] * inv * w[i];
        x[i] = v;
        if (conv_out) {
            const float* wc = conv_w + (size_t)i * conv_taps;
            float acc = 0.f;
            for (int j = 0; j < R; ++j) {
                const int src = p - (R - j);
                if (src >= 0) acc = fmaf(wc[j], st[(size_t)(src % R) * H + i], acc);
            }
            acc = fmaf(wc[R], v, acc);
            conv_out[(size_t)t * H + i] = from_float<TO>(acc + v);
        }
    }
}

extern "C" int scaled_add_rmsnorm(float* resid, const void* delta, int delta_dtype, float alpha, const float* w, float eps,
                                  const int* meta, int n, int H, float* keep, int keep_taps, long long keep_stride,
                                  long long conv_stride, const int* positions,
                                  const int* token_entry, const int* cu_tokens, const int* slots, const float* conv_w,
                                  const float* conv_state, int conv_taps, void* conv_out, int conv_out_dtype,
                                  cudaStream_t stream) {
    if (n <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    const size_t smem = (size_t)H * sizeof(float);
    if (keep_taps <= 1) keep = nullptr;
#define POSTNORM_CASE(TD, TO) \
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, scaled_add_rmsnorm_kernel<TD, TO>, n, threads, smem, stream, resid, \
                                  (const TD*)delta, alpha, w, eps, meta, H, keep, keep_taps - 1, keep_stride, conv_stride, positions, token_entry, \
                                  cu_tokens, slots, conv_w, conv_state, conv_taps, (TO*)conv_out)
    if (delta_dtype == DT_F32 && conv_out_dtype == DT_F32) POSTNORM_CASE(float, float);
    else if (delta_dtype == DT_F32) POSTNORM_CASE(float, __nv_bfloat16);
    else if (conv_out_dtype == DT_F32) POSTNORM_CASE(__nv_bfloat16, float);
    else POSTNORM_CASE(__nv_bfloat16, __nv_bfloat16);
#undef POSTNORM_CASE
}

// ----------------------------------------------------------------------------- attention rows
// One row of the fused projection per token: [q (nq heads of d) | k (nkv heads of d) | v (nkv heads of dv)].
//  * biases (q|k|v in one vector) are added;
//  * with q_norm / k_norm: the whole q part, and the whole k part, is divided by its root mean square (eps inside
//    the root) and multiplied by a weight of the part's size, before the rotation;
//  * the first `rot` dims of every q and k head rotate by position * inv_freq[i], dimension i with i + rot/2;
//  * with v_first: v <- (1 - lambda) v + lambda v_first (the same token's values of an earlier layer, rows of
//    nkv * dv); with v_out: the layer's values (biases added) are left there for later layers;
//  * q goes to q_out [T, nq, dp], k and v to the token's slot of its page, heads of dp elements (dp >= d, dv;
//    the tail is zeros, so that kernels that use one head size for keys and values can read them).
template <typename T>
__global__ void __launch_bounds__(256)
qkv_prepare_kernel(const T* __restrict__ qkv, const float* __restrict__ bias, const float* __restrict__ q_norm,
                   const float* __restrict__ k_norm, float eps, const int* __restrict__ positions,
                   const int* __restrict__ token_entry, const int* __restrict__ meta, int group,
                   const float* __restrict__ inv_freq, int rot, const T* __restrict__ v_first,
                   const float* __restrict__ v_lambda, T* __restrict__ v_out, T* __restrict__ q_out,
                   T* __restrict__ cache, int nq, int nkv, int d, int dv, int dp, int page_size, int num_pages,
                   int store_kv, int* __restrict__ status) {
    extern __shared__ float vals[];  // the q and k parts of the row, then cos[rot / 2], sin[rot / 2] of the token
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int NQ = nq * d, NK = nkv * d, NV = nkv * dv;
    const T* row = qkv + (size_t)t * (NQ + NK + NV);
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < NQ + NK; i += blockDim.x) {
        const float v = to_float(row[i]) + (bias ? bias[i] : 0.f);
        vals[i] = v;
        if (i < NQ) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
    }
    float inv_q = 1.f, inv_k = 1.f;
    if (q_norm) inv_q = rsqrtf(block_sum(sq, red) / (float)NQ + eps);
    if (k_norm) inv_k = rsqrtf(block_sum(sk, red) / (float)NK + eps);
    const int pos = positions[t], half = rot / 2;
    float* trig = vals + NQ + NK;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &trig[half + i], &trig[i]);
    int page = 0;
    if (store_kv) {
        const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group];
        page = bt[pos / page_size];
        if (page <= 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
            page = 0;  // keys and values are dropped; the queries are still prepared
        }
    }
    __syncthreads();
    const int slot = pos % page_size;
    const size_t head_block = (size_t)page_size * dp, kv_block = (size_t)nkv * head_block;
    T* kpage = cache + (size_t)page * 2 * kv_block + (size_t)slot * dp;
    T* vpage = kpage + kv_block;
    // q and k: one item per (head, dim below dp); pairs of the rotated part are computed twice, once per half
    const int heads = nq + (page > 0 ? nkv : 0);
    for (int it = threadIdx.x; it < heads * dp; it += blockDim.x) {
        const int h = it / dp, i = it % dp;
        const bool is_q = h < nq;
        T* dst = is_q ? q_out + ((size_t)t * nq + h) * dp : kpage + (size_t)(h - nq) * head_block;
        float r = 0.f;
        if (i < d) {
            const int base = h * d;  // k heads follow the q heads in vals
            const float inv = is_q ? inv_q : inv_k;
            const float* nw = is_q ? q_norm : k_norm;
            const int nb = is_q ? base : base - NQ;
            auto normed = [&](int j) { return vals[base + j] * inv * (nw ? nw[nb + j] : 1.f); };
            if (i < rot) {
                const int f = i < half ? i : i - half;
                float lo, hi;
                rotate_pair(normed(f), normed(f + half), trig[f], trig[half + f], lo, hi);
                r = i < half ? lo : hi;
            } else {
                r = normed(i);
            }
        }
        dst[i] = from_float<T>(r);
    }
    // values
    const float lam = (v_first && v_lambda) ? *v_lambda : 0.f;
    for (int it = threadIdx.x; it < nkv * dp; it += blockDim.x) {
        const int h = it / dp, i = it % dp;
        float r = 0.f;
        if (i < dv) {
            const int j = h * dv + i;
            r = to_float(row[NQ + NK + j]) + (bias ? bias[NQ + NK + j] : 0.f);
            if (v_out) v_out[(size_t)t * NV + j] = from_float<T>(r);
            if (v_first) r = (1.f - lam) * r + lam * to_float(v_first[(size_t)t * NV + j]);
        }
        if (page > 0) vpage[(size_t)h * head_block + i] = from_float<T>(r);
    }
}

extern "C" int qkv_prepare(const void* qkv, int dtype, const float* bias, const float* q_norm, const float* k_norm, float eps,
                           const int* positions, const int* token_entry, const int* meta, int group, const float* inv_freq,
                           int rot, const void* v_first, const float* v_lambda, void* v_out, void* q_out, void* cache, int T,
                           int nq, int nkv, int d, int dv, int dp, int page_size, int num_pages, int store_kv, int* status,
                           cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t smem = ((size_t)(nq + nkv) * d + rot) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = (nq + nkv) * d >= 1024 ? 256 : 128;
    cudaError_t e;
    static size_t configured[2] = {0, 0};  // the attribute only ever grows (and is not set inside a capture again)
#define PREP_CASE(TT, which) \
    do { \
        if (smem > 48 * 1024 && smem > configured[which]) { \
            e = cudaFuncSetAttribute(qkv_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured[which] = smem; \
        } \
        return (int)launch_kernel(qkv_prepare_kernel<TT>, T, threads, smem, stream, (const TT*)qkv, bias, q_norm, k_norm, eps, \
                                  positions, token_entry, meta, group, inv_freq, rot, (const TT*)v_first, v_lambda, (TT*)v_out, \
                                  (TT*)q_out, (TT*)cache, nq, nkv, d, dv, dp, page_size, num_pages, store_kv, status); \
    } while (0)
    if (dtype == DT_F32) PREP_CASE(float, 0);
    PREP_CASE(__nv_bfloat16, 1);
#undef PREP_CASE
}

// ----------------------------------------------------------------------------- polynomial activation of normalised powers
// out[t] = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u / sqrt(mean(u^2) + eps) over the row; powers element by
// element; coef = (a, b, c, e).  The three mean squares are sums of z^2, z^4 and z^6, taken in one pass.
template <typename T>
__global__ void __launch_bounds__(256)
polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ out,
                const int* __restrict__ meta, int F) {
    __shared__ float red[33];
    const float a = coef[0], b = coef[1], c = coef[2], e0 = coef[3];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (meta && t >= meta[META_NUM_TOKENS]) return;
    const T* zr = z + (size_t)t * F;
    T* o = out + (size_t)t * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = to_float(zr[i]), v2 = v * v, v3 = v2 * v;
        s2 += v2;
        s4 = fmaf(v2, v2, s4);
        s6 = fmaf(v3, v3, s6);
    }
    s2 = block_sum(s2, red);
    s4 = block_sum(s4, red);
    s6 = block_sum(s6, red);
    const float n1 = a * rsqrtf(s2 / (float)F + eps), n2 = b * rsqrtf(s4 / (float)F + eps), n3 = c * rsqrtf(s6 / (float)F + eps);
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = to_float(zr[i]), v2 = v * v;
        o[i] = from_float<T>(n1 * v + n2 * v2 + n3 * (v2 * v) + e0);
    }
}

extern "C" int polynorm(const void* z, int dtype, const float* coef, float eps, void* out, const int* meta, int T, int F,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = F >= 1024 ? 256 : 128;
    if (dtype == DT_F32)
        return (int)launch_kernel(polynorm_kernel<float>, T, threads, 0, stream, (const float*)z, coef, eps, (float*)out, meta, F);
    return (int)launch_kernel(polynorm_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)z, coef, eps,
                              (__nv_bfloat16*)out, meta, F);
}
