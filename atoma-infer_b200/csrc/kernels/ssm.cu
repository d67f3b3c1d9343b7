// Kernels of a state-space mixer of the Mamba-2 kind: the short causal convolution with bias and activation in
// front of the recurrence, the recurrence itself (sequential over a request's tokens, or cut into chunks of time that
// run side by side), and the gated norm in equal parts behind it.  Storage is float32 or bfloat16; the recurrence,
// its step sizes and decays, the gate and the norm are float32 always.
#include "common.cuh"

// ----------------------------------------------------------------------------- causal convolution, bias, activation
// y[t, c] = act(bias[c] + sum_j w[j, c] * u[t - taps + 1 + j, c]) over the rows of each request, zeros before its
// start.  u is a slice of a wider row (u_stride elements from row to row); w is [taps, C].  Rows before the step's
// portion come from the request's state: a ring of R = taps - 1 float32 rows per state slot (slot_stride floats from
// one slot to the next), the row of position p at ring place p mod R.  The ring is written by causal_conv_save AFTER
// this kernel has read it.  act 0: none; 1: SiLU.
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_act_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ w,
                       const float* __restrict__ bias, const float* __restrict__ state, long long slot_stride,
                       T* __restrict__ y, const int* __restrict__ meta, const int* __restrict__ positions,
                       const int* __restrict__ token_entry, const int* __restrict__ cu_tokens,
                       const int* __restrict__ slots, int C, int taps, int act) {
    // The step's metadata is written by no kernel of the step: it is read before the wait, while the kernel ahead ends.
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    const int e = live ? token_entry[t] : 0, p = live ? positions[t] : 0, first = live ? cu_tokens[e] : 0, R = taps - 1;
    const float* st = state ? state + (size_t)(live ? slots[e] : 0) * slot_stride : nullptr;
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = bias ? bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {  // oldest tap first: a fixed order
            const int back = taps - 1 - j, src = p - back;
            if (src < 0) continue;
            const float v = (t - back >= first) ? to_float(u[(size_t)(t - back) * u_stride + c]) : st[(size_t)(src % R) * C + c];
            acc = fmaf(w[(size_t)j * C + c], v, acc);
        }
        if (act == 1) acc = acc / (1.f + expf(-acc));
        y[(size_t)t * C + c] = from_float<T>(acc);
    }
}

// The same, V channels a thread with 16-byte accesses (V = 4 for float32, 8 for bfloat16; C, u_stride and slot_stride
// multiples of V, buffers on 16 bytes), the channels of a row dealt out over blocks (grid y).  save_own: every entry of
// the step brings one token, so the thread that read a channel's ring also writes the new row's place (p mod R, whose old
// row, of position p - R, it has just read): the ring is updated here and causal_conv_save is not needed.
template <typename T, int V>
__global__ void __launch_bounds__(128)
causal_conv_act_vec_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ w,
                           const float* __restrict__ bias, float* __restrict__ state, long long slot_stride,
                           T* __restrict__ y, const int* __restrict__ meta, const int* __restrict__ positions,
                           const int* __restrict__ token_entry, const int* __restrict__ cu_tokens,
                           const int* __restrict__ slots, int C, int taps, int act, int save_own) {
    const int t = blockIdx.x, c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const bool live = t < meta[META_NUM_TOKENS] && c < C;
    const int e = live ? token_entry[t] : 0, p = live ? positions[t] : 0, first = live ? cu_tokens[e] : 0, R = taps - 1;
    float* st = state ? state + (size_t)(live ? slots[e] : 0) * slot_stride : nullptr;
    float acc[V];
    if (live) {  // weights and bias depend on no earlier kernel: fetched before the wait
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            float b4[4] = {0.f, 0.f, 0.f, 0.f};
            if (bias) load4(bias + c + i, b4);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[i + k] = b4[k];
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    float cur[V];
    for (int j = 0; j < taps; ++j) {  // oldest tap first: a fixed order
        const int back = taps - 1 - j, src = p - back;
        if (src < 0) continue;
        float v[V], wv[V];
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            float t4[4], w4[4];
            if (t - back >= first) load4(u + (size_t)(t - back) * u_stride + c + i, t4);
            else load4(st + (size_t)(src % R) * C + c + i, t4);
            load4(w + (size_t)j * C + c + i, w4);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[i + k] = t4[k], wv[i + k] = w4[k];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(wv[i], v[i], acc[i]);
        if (back == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i) cur[i] = v[i];
        }
    }
    if (act == 1) {
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = acc[i] / (1.f + expf(-acc[i]));
    }
#pragma unroll
    for (int i = 0; i < V; i += 4) {
        const float o4[4] = {acc[i], acc[i + 1], acc[i + 2], acc[i + 3]};
        store4(y + (size_t)t * C + c + i, o4);
    }
    if (save_own && R > 0) {
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            const float s4[4] = {cur[i], cur[i + 1], cur[i + 2], cur[i + 3]};
            store4(st + (size_t)(p % R) * C + c + i, s4);
        }
    }
}

extern "C" int causal_conv_act(const void* u, int dtype, long long u_stride, const float* w, const float* bias,
                               float* state, long long slot_stride, void* y, const int* meta, const int* positions,
                               const int* token_entry, const int* cu_tokens, const int* slots, int T, int C, int taps,
                               int act, int save_own, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (taps < 1 || (taps > 1 && !state)) return (int)cudaErrorInvalidValue;
    const int V = dtype == DT_F32 ? 4 : 8;
    if (C % V == 0 && u_stride % V == 0 && slot_stride % 4 == 0 &&
        (((uintptr_t)u | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)state | (uintptr_t)y) & 15) == 0) {
        dim3 grid(T, (C / V + 127) / 128);
        if (dtype == DT_F32)
            return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, causal_conv_act_vec_kernel<float, 4>, grid, 128, 0, stream,
                                          (const float*)u, u_stride, w, bias, (float*)state, slot_stride, (float*)y, meta, positions,
                                          token_entry, cu_tokens, slots, C, taps, act, save_own);
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, causal_conv_act_vec_kernel<__nv_bfloat16, 8>, grid, 128, 0, stream,
                                      (const __nv_bfloat16*)u, u_stride, w, bias, (float*)state, slot_stride, (__nv_bfloat16*)y, meta,
                                      positions, token_entry, cu_tokens, slots, C, taps, act, save_own);
    }
    if (save_own) return (int)cudaErrorInvalidValue;  // (ask causal_conv_act_saves first)
    const int threads = C >= 1024 ? 256 : 128;
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, causal_conv_act_kernel<float>, T, threads, 0, stream, (const float*)u,
                                      u_stride, w, bias, state, slot_stride, (float*)y, meta, positions, token_entry, cu_tokens,
                                      slots, C, taps, act);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, causal_conv_act_kernel<__nv_bfloat16>, T, threads, 0, stream,
                                  (const __nv_bfloat16*)u, u_stride, w, bias, state, slot_stride, (__nv_bfloat16*)y, meta,
                                  positions, token_entry, cu_tokens, slots, C, taps, act);
}

// Whether causal_conv_act can update the ring itself (see save_own) for these sizes and addresses.
extern "C" int causal_conv_act_saves(const void* u, int dtype, long long u_stride, const float* w, const float* bias,
                                     const float* state, long long slot_stride, const void* y, int C) {
    const int V = dtype == DT_F32 ? 4 : 8;
    return C % V == 0 && u_stride % V == 0 && slot_stride % 4 == 0 &&
           (((uintptr_t)u | (uintptr_t)w | (uintptr_t)bias | (uintptr_t)state | (uintptr_t)y) & 15) == 0;
}

// The last R rows of u of every entry go to its ring.
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_save_kernel(const T* __restrict__ u, long long u_stride, float* __restrict__ state, long long slot_stride,
                        const int* __restrict__ meta, const int* __restrict__ positions, const int* __restrict__ token_entry,
                        const int* __restrict__ cu_tokens, const int* __restrict__ slots, int C, int R) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int e = token_entry[t];
    if (t < cu_tokens[e + 1] - R) return;
    float* st = state + (size_t)slots[e] * slot_stride + (size_t)(positions[t] % R) * C;
    for (int c = threadIdx.x; c < C; c += blockDim.x) st[c] = to_float(u[(size_t)t * u_stride + c]);
}

extern "C" int causal_conv_save(const void* u, int dtype, long long u_stride, float* state, long long slot_stride,
                                const int* meta, const int* positions, const int* token_entry, const int* cu_tokens,
                                const int* slots, int T, int C, int taps, cudaStream_t stream) {
    if (T <= 0 || taps <= 1) return 0;
    const int threads = C >= 1024 ? 256 : 128;
    if (dtype == DT_F32)
        return (int)launch_kernel(causal_conv_save_kernel<float>, T, threads, 0, stream, (const float*)u, u_stride, state,
                                  slot_stride, meta, positions, token_entry, cu_tokens, slots, C, taps - 1);
    return (int)launch_kernel(causal_conv_save_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)u, u_stride,
                              state, slot_stride, meta, positions, token_entry, cu_tokens, slots, C, taps - 1);
}

// ----------------------------------------------------------------------------- the recurrence
// Per head h (of group h / (heads / groups)) a matrix S of N x P: S_t = exp(-exp(a_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T,
// y_t = S_t^T C_t + d_h x_t, dt_t = softplus(raw_t + dt_bias_h).  Rows of `xbc` are [x: heads * P | B: groups * N |
// C: groups * N]; `dt` is a slice of a wider row.
//
// One block per (head, entry[, chunk]).  Thread (p, r) keeps NPT rows n = r * NPT .. of column p in registers, R
// threads share a column (R * NPT >= N; rows beyond N see B = C = 0 and stay zero).  Tokens come through shared
// memory SCAN_TT at a time; y_t is summed over a thread's rows in order, then over the R threads by shuffles: an order
// that depends on the sizes only.
//
// pass 0: the entry's tokens in order, from the state slot, y written, the slot updated.
// Cut into chunks of `chunk_len` tokens (counted from the entry's first token in the step), three launches:
// pass 1: chunk c < last runs from S = 0 and leaves its end state in scratch[c + 1] and its total decay in decay[c];
// (ssm_chunk_states) scratch[0] = slot's state, scratch[c] = decay[c - 1] * scratch[c - 1] + scratch[c], in order;
// pass 3: chunk c runs again from scratch[c] and writes y; the last chunk updates the slot.
#define SCAN_TT 16

// Eight (bfloat16) or four (float32) consecutive elements of a row, widened, into shared memory.
__device__ __forceinline__ void stage8(const __nv_bfloat16* src, float* dst) {
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
    *reinterpret_cast<float4*>(dst) = make_float4(a.x, a.y, b.x, b.y);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(c.x, c.y, d.x, d.y);
}
__device__ __forceinline__ void stage8(const float* src, float* dst) {
    *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
    *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
}

// BIG: blocks of more than 256 threads (at most 128 registers a thread; else up to 255, which 64 rows of state with their
// loads in flight need to stay out of local memory).
template <typename T, int NPT, bool WRITE_Y, bool BIG>
__global__ void __launch_bounds__(BIG ? 512 : 256)
ssm_scan_kernel(const T* __restrict__ xbc, int xbc_stride, const T* __restrict__ dt, long long dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, long long slot_stride, float* __restrict__ y, const int* __restrict__ meta,
                const int* __restrict__ cu_tokens, const int* __restrict__ slots, int heads, int P, int N, int groups, int R,
                int pass, int chunk_len, int max_chunks, float* __restrict__ scratch, float* __restrict__ decay, int vec8) {
    extern __shared__ __align__(16) float sm[];
    // A token's B (and C) in shared memory: R slices of NPT rows, one a thread of a column; with several slices each
    // starts four floats later than the rows alone would put it, so that the R addresses a warp reads at once fall
    // into different banks.  Row n lies at (n / NPT) * SL + n % NPT.
    const int SL = R > 1 ? NPT + 4 : NPT, NL = R * NPT, NP = R * SL;
    float* Bs = sm;                         // [SCAN_TT][NP]
    float* Cs = Bs + SCAN_TT * NP;          // [SCAN_TT][NP]
    float* xs = Cs + SCAN_TT * NP;          // [SCAN_TT][P]
    float* dts = xs + SCAN_TT * P;          // [SCAN_TT]
    float* decs = dts + SCAN_TT;            // [SCAN_TT]
    const int h = blockIdx.x, e = blockIdx.y, c = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int first = cu_tokens[e], count = cu_tokens[e + 1] - first;
    const int nchunks = pass == 0 ? 1 : (count + chunk_len - 1) / chunk_len;
    if (c >= nchunks || (pass == 1 && c == nchunks - 1)) return;
    const int t0 = first + (pass == 0 ? 0 : c * chunk_len), t1 = pass == 0 ? first + count : min(first + count, t0 + chunk_len);
    const int tid = threadIdx.x, p = tid / R, r = tid % R;
    const bool real = p < P;
    const int inner = heads * P, g = h / (heads / groups);
    const float rate = expf(a_log[h]), bias = dt_bias[h], dskip = d_skip[h];
    const size_t HS = (size_t)N * P;        // floats of one head's matrix
    float* slot_state = state + (size_t)slots[e] * slot_stride + (size_t)h * HS;
    float* chunk_state = scratch ? scratch + (((size_t)e * max_chunks + c) * heads + h) * HS : nullptr;

    float S[NPT];
    const float* init = pass == 0 ? slot_state : (pass == 3 ? chunk_state : nullptr);
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = r * NPT + i;
        S[i] = (init && real && n < N) ? init[(size_t)n * P + p] : 0.f;
    }
    float dt_sum = 0.f;
    for (int tb = t0; tb < t1; tb += SCAN_TT) {
        const int nt = min(SCAN_TT, t1 - tb);
        __syncthreads();  // the previous tile is no longer read
        if (vec8) {  // a warp a row, a lane eight elements a step: every load of the tile is in flight at once
            const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
            for (int tt = warp; tt < nt; tt += nwarps) {
                const T* row = xbc + (size_t)(tb + tt) * xbc_stride;
                const T* brow = row + inner + (size_t)g * N;
                for (int n = lane * 8; n < NL; n += 256) {
                    const int at = tt * NP + (n / NPT) * SL + n % NPT;
                    if (n < N) {
                        stage8(brow + n, Bs + at);
                        stage8(brow + (size_t)groups * N + n, Cs + at);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) Bs[at + i] = Cs[at + i] = 0.f;
                    }
                }
                for (int q = lane * 8; q < P; q += 256) stage8(row + (size_t)h * P + q, xs + tt * P + q);
            }
        } else {
            for (int idx = tid; idx < nt * NL; idx += blockDim.x) {
                const int tt = idx / NL, n = idx % NL, at = tt * NP + (n / NPT) * SL + n % NPT;
                const T* row = xbc + (size_t)(tb + tt) * xbc_stride + inner + (size_t)g * N;
                Bs[at] = n < N ? to_float(row[n]) : 0.f;
                Cs[at] = n < N ? to_float(row[(size_t)groups * N + n]) : 0.f;
            }
            for (int idx = tid; idx < nt * P; idx += blockDim.x) {
                const int tt = idx / P, q = idx % P;
                xs[idx] = to_float(xbc[(size_t)(tb + tt) * xbc_stride + (size_t)h * P + q]);
            }
        }
        if (tid < nt) {
            const float raw = to_float(dt[(size_t)(tb + tid) * dt_stride + h]) + bias;
            const float step = raw > 20.f ? raw : log1pf(expf(raw));  // softplus; beyond 20 the difference is below rounding
            dts[tid] = step;
            decs[tid] = expf(-rate * step);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float xv = real ? xs[tt * P + p] : 0.f, step = dts[tt], dec = decs[tt];
            const float dx = step * xv;
            const float* Bt = Bs + tt * NP + r * SL;
            const float* Ct = Cs + tt * NP + r * SL;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPT; i += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(Bt + i);
                S[i] = fmaf(dec, S[i], b4.x * dx);
                S[i + 1] = fmaf(dec, S[i + 1], b4.y * dx);
                S[i + 2] = fmaf(dec, S[i + 2], b4.z * dx);
                S[i + 3] = fmaf(dec, S[i + 3], b4.w * dx);
                if (WRITE_Y) {
                    const float4 c4 = *reinterpret_cast<const float4*>(Ct + i);
                    acc = fmaf(S[i], c4.x, acc);
                    acc = fmaf(S[i + 1], c4.y, acc);
                    acc = fmaf(S[i + 2], c4.z, acc);
                    acc = fmaf(S[i + 3], c4.w, acc);
                }
            }
            if (WRITE_Y) {
                for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (real && r == 0) y[(size_t)(tb + tt) * inner + (size_t)h * P + p] = fmaf(dskip, xv, acc);
            }
            dt_sum += step;
        }
    }
    float* fin = pass == 1 ? chunk_state + (size_t)heads * HS /* scratch[c + 1] */ : ((pass == 0 || c == nchunks - 1) ? slot_state : nullptr);
    if (fin && real) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = r * NPT + i;
            if (n < N) fin[(size_t)n * P + p] = S[i];
        }
    }
    if (pass == 1 && tid == 0) decay[((size_t)e * max_chunks + c) * heads + h] = expf(-rate * dt_sum);
}

// scratch[e, 0] = the slot's state; scratch[e, c] = decay[e, c - 1] * scratch[e, c - 1] + scratch[e, c] for c = 1 ..
__global__ void __launch_bounds__(256)
ssm_chunk_states_kernel(const float* __restrict__ state, long long slot_stride, float* __restrict__ scratch,
                        const float* __restrict__ decay, const int* __restrict__ meta, const int* __restrict__ cu_tokens,
                        const int* __restrict__ slots, int heads, long long HS, int chunk_len, int max_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int count = cu_tokens[e + 1] - cu_tokens[e], nchunks = (count + chunk_len - 1) / chunk_len;
    const float* src = state + (size_t)slots[e] * slot_stride + (size_t)h * HS;
    for (long long i = (long long)blockIdx.z * blockDim.x + threadIdx.x; i < HS; i += (long long)gridDim.z * blockDim.x) {
        float s = src[i];
        scratch[(((size_t)e * max_chunks) * heads + h) * HS + i] = s;
        for (int c = 1; c < nchunks; ++c) {
            float* at = scratch + (((size_t)e * max_chunks + c) * heads + h) * HS + i;
            s = fmaf(decay[((size_t)e * max_chunks + c - 1) * heads + h], s, *at);
            *at = s;
        }
    }
}

// The most rows of state a thread keeps (a lever for measurements; 64: all instantiations).
static int g_scan_max_rows = 64;
extern "C" void ssm_scan_set_max_rows(int n) { g_scan_max_rows = n; }

// How a head's N rows are dealt out: R threads a column, NPT rows a thread (R * NPT >= N, R a power of two).
static bool scan_geometry(int N, int P, int* R_out, int* NPT_out) {
    static const int sizes[] = {16, 24, 32, 48, 64};
    int best_r = 0, best_npt = 0;
    long best_cost = -1;
    for (int R = 1; R <= 32; R *= 2) {
        const int threads = ((P * R + 31) / 32) * 32;
        if (threads > 512) break;
        for (int k = 0; k < 5; ++k) {
            const int npt = sizes[k];
            if (R * npt < N || npt > g_scan_max_rows) continue;
            const long cost = (long)R * npt * 8 + (R > 1 ? R : 0);  // padded work first, then the fewest threads a column
            if (best_cost < 0 || cost < best_cost) best_cost = cost, best_r = R, best_npt = npt;
            break;
        }
    }
    if (best_cost < 0) return false;
    *R_out = best_r;
    *NPT_out = best_npt;
    return true;
}

extern "C" size_t ssm_scan_scratch_floats(int S, int heads, int P, int N, int max_chunks) {
    return (size_t)S * max_chunks * heads * ((size_t)N * P + 1);
}

template <typename T>
static int ssm_scan_launch(int NPT, dim3 grid, int threads, size_t smem, cudaStream_t stream, const T* xbc, int xbc_stride,
                           const T* dt, long long dt_stride, const float* dt_bias, const float* a_log, const float* d_skip,
                           float* state, long long slot_stride, float* y, const int* meta, const int* cu_tokens,
                           const int* slots, int heads, int P, int N, int groups, int R, int pass, int chunk_len,
                           int max_chunks, float* scratch, float* decay) {
    // eight elements a load: rows of x, B and C that start on 16 bytes (float32: two loads of four)
    const int vec8 = P % 8 == 0 && N % 8 == 0 && xbc_stride % 8 == 0 && ((uintptr_t)xbc & 15) == 0 && (R * NPT) % 8 == 0;
#define SCAN_CASE(K, Y, B)                                                                                                  \
    case K: {                                                                                                              \
        static size_t configured = 0;                                                                                      \
        if (smem > 48 * 1024 && smem > configured) {                                                                       \
            cudaError_t err = cudaFuncSetAttribute(ssm_scan_kernel<T, K, Y, B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (err != cudaSuccess) return (int)err;                                                                       \
            configured = smem;                                                                                             \
        }                                                                                                                  \
        return (int)launch_kernel(ssm_scan_kernel<T, K, Y, B>, grid, threads, smem, stream, xbc, xbc_stride, dt, dt_stride, dt_bias, \
                                  a_log, d_skip, state, slot_stride, y, meta, cu_tokens, slots, heads, P, N, groups, R, pass,  \
                                  chunk_len, max_chunks, scratch, decay, vec8);                                            \
    }
#define SCAN_SIZES(Y, B) switch (NPT) { SCAN_CASE(16, Y, B) SCAN_CASE(24, Y, B) SCAN_CASE(32, Y, B) SCAN_CASE(48, Y, B) SCAN_CASE(64, Y, B) }
    if (pass == 1) {  // chunks that only leave their end state: no y, a third less arithmetic
        if (threads > 256) SCAN_SIZES(false, true) else SCAN_SIZES(false, false)
    } else {
        if (threads > 256) SCAN_SIZES(true, true) else SCAN_SIZES(true, false)
    }
#undef SCAN_SIZES
#undef SCAN_CASE
    return (int)cudaErrorInvalidValue;
}

// chunk_len 0: every entry's tokens in order (one launch); else the three launches described above, with
// `scratch` of ssm_scan_scratch_floats(S, ..., max_chunks) floats, max_chunks >= the chunks of the longest entry.
extern "C" int ssm_scan(const void* xbc, int dtype, int xbc_stride, const void* dt, long long dt_stride, const float* dt_bias,
                        const float* a_log, const float* d_skip, float* state, long long slot_stride, float* y,
                        const int* meta, const int* cu_tokens, const int* slots, int S, int heads, int P, int N, int groups,
                        int chunk_len, int max_chunks, float* scratch, cudaStream_t stream) {
    if (S <= 0) return 0;
    int R = 0, NPT = 0;
    if (heads % groups || !scan_geometry(N, P, &R, &NPT)) return (int)cudaErrorInvalidValue;
    const int threads = ((P * R + 31) / 32) * 32;
    const size_t smem = (size_t)(2 * SCAN_TT * R * (R > 1 ? NPT + 4 : NPT) + SCAN_TT * P + 2 * SCAN_TT) * sizeof(float);
    float* decay = scratch ? scratch + (size_t)S * max_chunks * heads * (size_t)N * P : nullptr;
#define SCAN_PASS(TT, pass, chunks)                                                                                        \
    ssm_scan_launch<TT>(NPT, dim3(heads, S, chunks), threads, smem, stream, (const TT*)xbc, xbc_stride, (const TT*)dt, dt_stride, \
                        dt_bias, a_log, d_skip, state, slot_stride, y, meta, cu_tokens, slots, heads, P, N, groups, R, pass, \
                        chunk_len, max_chunks, scratch, decay)
    if (chunk_len <= 0 || max_chunks <= 1 || !scratch)
        return dtype == DT_F32 ? SCAN_PASS(float, 0, 1) : SCAN_PASS(__nv_bfloat16, 0, 1);
    int err = dtype == DT_F32 ? SCAN_PASS(float, 1, max_chunks) : SCAN_PASS(__nv_bfloat16, 1, max_chunks);
    if (err) return err;
    const long long HS = (long long)N * P;
    const int zblocks = (int)((HS + 1023) / 1024);
    err = (int)launch_kernel(ssm_chunk_states_kernel, dim3(heads, S, zblocks), 256, 0, stream, (const float*)state, slot_stride,
                             scratch, (const float*)decay, meta, cu_tokens, slots, heads, HS, chunk_len, max_chunks);
    if (err) return err;
    return dtype == DT_F32 ? SCAN_PASS(float, 3, max_chunks) : SCAN_PASS(__nv_bfloat16, 3, max_chunks);
#undef SCAN_PASS
}

// ----------------------------------------------------------------------------- gate, then the norm in equal parts
// v = y * silu(z); out = v / sqrt(mean(v^2) + eps) * w, the mean taken over each of `parts` equal parts of the row.
// y is float32 [T, n]; z a slice of a wider row.  One block per (token, part).
template <typename T>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride, const float* __restrict__ w,
                        float eps, T* __restrict__ out, const int* __restrict__ meta, int n, int parts, int vec4) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x, part = blockIdx.y, len = n / parts, at = part * len;
    if (t >= meta[META_NUM_TOKENS]) return;
    const float* yr = y + (size_t)t * n + at;
    const T* zr = z + (size_t)t * z_stride + at;
    float ss = 0.f;
    if (vec4 && len <= 8 * (int)blockDim.x) {  // the same, four consecutive values a thread and 16-byte accesses
        float v[2][4];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) v[k][j] = 0.f;
            if (i < len) {
                float yv[4], zv[4];
                load4(yr + i, yv);
                load4(zr + i, zv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[k][j] = yv[j] * (zv[j] / (1.f + expf(-zv[j])));
                    ss = fmaf(v[k][j], v[k][j], ss);
                }
            }
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)len + eps);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = (threadIdx.x + k * blockDim.x) * 4;
            if (i < len) {
                float wv[4];
                load4(w + at + i, wv);
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[j] = v[k][j] * inv * wv[j];
                store4(out + (size_t)t * n + at + i, wv);
            }
        }
        return;
    }
    if (len <= 8 * (int)blockDim.x) {  // the gated values wait in registers for the sum: y and z are read once
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            v[k] = 0.f;
            if (i < len) {
                const float g = to_float(zr[i]);
                v[k] = yr[i] * (g / (1.f + expf(-g)));
            }
            ss = fmaf(v[k], v[k], ss);
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)len + eps);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int i = threadIdx.x + k * blockDim.x;
            if (i < len) out[(size_t)t * n + at + i] = from_float<T>(v[k] * inv * w[at + i]);
        }
        return;
    }
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float g = to_float(zr[i]);
        const float v = yr[i] * (g / (1.f + expf(-g)));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)len + eps);
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float g = to_float(zr[i]);
        const float v = yr[i] * (g / (1.f + expf(-g)));
        out[(size_t)t * n + at + i] = from_float<T>(v * inv * w[at + i]);
    }
}

extern "C" int gated_group_norm(const float* y, const void* z, int dtype, long long z_stride, const float* w, float eps,
                                void* out, const int* meta, int T, int n, int parts, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (parts <= 0 || n % parts) return (int)cudaErrorInvalidValue;
    const int len = n / parts, threads = len >= 1024 ? 256 : 128;
    // four values per access: parts and rows start on multiples of four elements and the buffers on 16 bytes
    const int vec4 = len % 4 == 0 && z_stride % 4 == 0 && (((uintptr_t)y | (uintptr_t)z | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, gated_group_norm_kernel<float>, dim3(T, parts), threads, 0, stream, y,
                                      (const float*)z, z_stride, w, eps, (float*)out, meta, n, parts, vec4);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, gated_group_norm_kernel<__nv_bfloat16>, dim3(T, parts), threads, 0, stream,
                                  y, (const __nv_bfloat16*)z, z_stride, w, eps, (__nv_bfloat16*)out, meta, n, parts, vec4);
}
