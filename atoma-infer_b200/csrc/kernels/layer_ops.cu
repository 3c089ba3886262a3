// Kernels of layers that are not the plain pre-norm block: a short causal convolution over time with its state,
// the norm that comes after the sum, the preparation of attention rows whose queries and keys are normalised as
// whole projections (with biases, a partial rotation and a mix of an earlier layer's values), and the polynomial
// activation of normalised powers.  float32 and bfloat16 storage alike; all arithmetic is float32, and every
// reduction runs in an order that depends only on the row it belongs to.
#include "common.cuh"

// N sums over a block at once, in the fixed order of block_sum (warp shuffles, then warp 0 over the warp sums), with two
// barriers for all of them.  `scratch` holds N * 33 floats in shared memory.  All threads get the results.
template <int N>
__device__ __forceinline__ void block_sums(float (&v)[N], float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = warp_sum(v[k]);
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < N; ++k) scratch[k * 33 + warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < N; ++k) {
            float t = lane < nwarps ? scratch[k * 33 + lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) scratch[k * 33 + 32] = t;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = scratch[k * 33 + 32];
}

// ----------------------------------------------------------------------------- short convolution over time
// What a sublayer reads: y[t] = x[t] * (1 or 0) + sum_j w[j, c] * x[t - taps + 1 + j], x the float32 residual
// stream, zeros before the start of a request; w is [taps, C] (the checkpoint's [C, taps] transposed once at load
// time), so that the threads of a warp read neighbouring weights.  Rows before the step's portion come from the request's state: a
// ring of R = taps - 1 rows per state slot (slot_stride floats from one slot to the next), the row of position p at
// ring place p mod R.  The state is written by
// short_conv_save (or by the norm kernel below) AFTER this kernel has read it: only the last R rows of an entry
// are written, and within a step they land on places whose old rows this kernel may still need.
template <typename TO>
__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ state,
                  TO* __restrict__ y, const int* __restrict__ meta, const int* __restrict__ positions,
                  const int* __restrict__ token_entry, const int* __restrict__ cu_tokens,
                  const int* __restrict__ slots, int C, int taps, int add_input, long long slot_stride, int vec4) {
    // The step's metadata is written by no kernel of the step: it is read before the wait, while the kernel ahead ends.
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    const int e = live ? token_entry[t] : 0, p = live ? positions[t] : 0, first = live ? cu_tokens[e] : 0, R = taps - 1;
    const float* st = state + (size_t)(live ? slots[e] : 0) * slot_stride;
    pdl_wait();  // like the norm kernel: the kernels behind start once this one's wait is over
    pdl_launch_dependents();
    if (!live) return;
    if (vec4) {  // four channels a thread, 16-byte accesses (C a multiple of 4, buffers on 16 bytes)
        for (int c = threadIdx.x * 4; c < C; c += blockDim.x * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < taps; ++j) {  // oldest tap first: a fixed order
                const int back = taps - 1 - j, src = p - back;
                if (src < 0) continue;
                float v[4], wv[4];
                load4((t - back >= first) ? x + (size_t)(t - back) * C + c : st + (size_t)(src % R) * C + c, v);
                load4(w + (size_t)j * C + c, wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] = fmaf(wv[i], v[i], acc[i]);
            }
            if (add_input) {
                float v[4];
                load4(x + (size_t)t * C + c, v);
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] += v[i];
            }
            store4(y + (size_t)t * C + c, acc);
        }
        return;
    }
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {  // oldest tap first: a fixed order
            const int back = taps - 1 - j, src = p - back;
            if (src < 0) continue;
            const float v = (t - back >= first) ? x[(size_t)(t - back) * C + c] : st[(size_t)(src % R) * C + c];
            acc = fmaf(w[(size_t)j * C + c], v, acc);
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
    const int vec4 = C % 4 == 0 && slot_stride % 4 == 0 && (((uintptr_t)x | (uintptr_t)state | (uintptr_t)y | (uintptr_t)w) & 15) == 0;
    if (y_dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, short_conv_kernel<float>, T, threads, 0, stream, x, w, state, (float*)y, meta, positions,
                                  token_entry, cu_tokens, slots, C, taps, add_input, slot_stride, vec4);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, short_conv_kernel<__nv_bfloat16>, T, threads, 0, stream, x, w, state, (__nv_bfloat16*)y, meta,
                              positions, token_entry, cu_tokens, slots, C, taps, add_input, slot_stride, vec4);
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
template <typename TD, typename TO, bool CONV>
__global__ void __launch_bounds__(256)
scaled_add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, float alpha, const float* __restrict__ w,
                          float eps, const int* __restrict__ meta, int H, float* __restrict__ keep, int keep_rows,
                          long long keep_stride, long long conv_stride,
                          const int* __restrict__ positions, const int* __restrict__ token_entry,
                          const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                          const float* __restrict__ conv_w, const float* __restrict__ conv_state, int conv_taps,
                          TO* __restrict__ conv_out_arg, int vec4) {
    TO* const conv_out = CONV ? conv_out_arg : nullptr;  // the plain instantiation keeps its registers
    __shared__ float red[33];
    extern __shared__ __align__(16) float row[];  // H floats, and H more with conv_out
    // The step's metadata is written by no kernel of the step: it is read before the wait, while the kernel ahead ends.
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    const int e = live && (keep || conv_out) ? token_entry[t] : 0;
    const int slot = live && (keep || conv_out) ? slots[e] : 0, my_pos = live && (keep || conv_out) ? positions[t] : 0;
    float* kept = nullptr;
    if (live && keep && keeps_row(t, e, cu_tokens, keep_rows))
        kept = keep + (size_t)slot * keep_stride + (size_t)(my_pos % keep_rows) * H;
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    float* x = resid + (size_t)t * H;
    const TD* dl = delta ? delta + (size_t)t * H : nullptr;
    // The part of the next sublayer's convolution that comes from its state does not depend on this norm: it is taken
    // in the first pass, with the loads of the row, and waits in shared memory behind the row.
    const int R = conv_taps - 1;
    const int p = my_pos;
    const float* st = conv_out ? conv_state + (size_t)slot * conv_stride : nullptr;
    float* pre = row + H;
    float ss = 0.f;
    if (vec4) {  // four values a thread, 16-byte accesses; the sum's order differs from the scalar form's, but is as fixed
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float old[4], d[4] = {0.f, 0.f, 0.f, 0.f}, v[4];
            load4(x + i, old);
            if (kept) store4(kept + i, old);
            if (dl) load4(dl + i, d);
            if (conv_out) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < R; ++j) {
                    const int src = p - (R - j);
                    if (src < 0) continue;
                    float sv[4], wv[4];
                    load4(st + (size_t)(src % R) * H + i, sv);
                    load4(conv_w + (size_t)j * H + i, wv);
#pragma unroll
                    for (int k = 0; k < 4; ++k) acc[k] = fmaf(wv[k], sv[k], acc[k]);
                }
                store4(pre + i, acc);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[k] = dl ? fmaf(alpha, old[k], d[k]) : alpha * old[k];
                ss = fmaf(v[k], v[k], ss);
            }
            store4(row + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float old = x[i];
            if (kept) kept[i] = old;
            if (conv_out) {
                float acc = 0.f;
                for (int j = 0; j < R; ++j) {
                    const int src = p - (R - j);
                    if (src >= 0) acc = fmaf(conv_w[(size_t)j * H + i], st[(size_t)(src % R) * H + i], acc);
                }
                pre[i] = acc;
            }
            const float v = dl ? fmaf(alpha, old, to_float(dl[i])) : alpha * old;
            row[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    if (vec4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4], wv[4];
            load4(row + i, v);
            load4(w + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = v[k] * inv * wv[k];
            store4(x + i, v);
            if (conv_out) {  // conv_w is [taps, H]; its last row is the tap of the new row itself
                float acc[4], cw[4];
                load4(pre + i, acc);
                load4(conv_w + (size_t)R * H + i, cw);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = fmaf(cw[k], v[k], acc[k]) + v[k];
                store4(conv_out + (size_t)t * H + i, acc);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = row[i] * inv * w[i];
        x[i] = v;
        if (conv_out) conv_out[(size_t)t * H + i] = from_float<TO>(fmaf(conv_w[(size_t)R * H + i], v, pre[i]) + v);
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
    const size_t smem = (size_t)H * sizeof(float) * (conv_out ? 2 : 1);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // per instantiation; grows only, and is not set inside a capture again
    if (keep_taps <= 1) keep = nullptr;
    const int vec4 = H % 4 == 0 && keep_stride % 4 == 0 && conv_stride % 4 == 0 &&
                     (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)keep | (uintptr_t)conv_w |
                       (uintptr_t)conv_state | (uintptr_t)conv_out) & 15) == 0;
#define POSTNORM_CASE(TD, TO, which) \
    if (conv_out) { POSTNORM_CASE2(TD, TO, true, 2 * which); } \
    POSTNORM_CASE2(TD, TO, false, 2 * which + 1)
#define POSTNORM_CASE2(TD, TO, CONV, which) \
    if (smem > 48 * 1024 && smem > configured[which]) { \
        cudaError_t e = cudaFuncSetAttribute(scaled_add_rmsnorm_kernel<TD, TO, CONV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return (int)e; \
        configured[which] = smem; \
    } \
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, scaled_add_rmsnorm_kernel<TD, TO, CONV>, n, threads, smem, stream, resid, \
                                  (const TD*)delta, alpha, w, eps, meta, H, keep, keep_taps - 1, keep_stride, conv_stride, positions, token_entry, \
                                  cu_tokens, slots, conv_w, conv_state, conv_taps, (TO*)conv_out, vec4)
    if (delta_dtype == DT_F32 && conv_out_dtype == DT_F32) { POSTNORM_CASE(float, float, 0); }
    else if (delta_dtype == DT_F32) { POSTNORM_CASE(float, __nv_bfloat16, 1); }
    else if (conv_out_dtype == DT_F32) { POSTNORM_CASE(__nv_bfloat16, float, 2); }
    else { POSTNORM_CASE(__nv_bfloat16, __nv_bfloat16, 3); }
#undef POSTNORM_CASE
#undef POSTNORM_CASE2
}

// ----------------------------------------------------------------------------- attention rows
// One row of the fused projection per token: [q (nq heads of d) | k (nkv heads of d) | v (nkv heads of dv)].
//  * biases (q|k|v in one vector) are added;
//  * with q_norm / k_norm: the whole q part, and the whole k part, is divided by its root mean square (eps inside
//    the root) and multiplied by a weight of the part's size, before the rotation;
//  * the first `rot` dims of every q and k head rotate by position * inv_freq[i], dimension i with i + rot/2;
//  * with head_norm: after the rotation every q head and every k head is divided by its own root mean square over d
//    (eps inside the root; no weight);
//  * with v_first: v <- (1 - lambda) v + lambda v_first (the same token's values of an earlier layer, rows of
//    nkv * dv); with v_out: the layer's values (biases added) are left there for later layers;
//  * q goes to q_out [T, nq, dp], k and v to the token's slot of its page, heads of dp elements (dp >= d, dv;
//    the tail is zeros, so that kernels that use one head size for keys and values can read them).
template <typename T, typename TP>
__global__ void __launch_bounds__(256)
qkv_prepare_kernel(const T* __restrict__ qkv, long long qkv_stride, const TP* __restrict__ bias_g, const TP* __restrict__ q_norm_g,
                   const TP* __restrict__ k_norm_g, float eps, const int* __restrict__ positions,
                   const int* __restrict__ token_entry, const int* __restrict__ meta, int group,
                   const float* __restrict__ inv_freq, int rot, const T* __restrict__ v_first,
                   const float* __restrict__ v_lambda, T* __restrict__ v_out, T* __restrict__ q_out,
                   T* __restrict__ cache, int nq, int nkv, int d, int dv, int dp, int page_size, int num_pages,
                   int store_kv, int vec4, int head_norm, int interleaved, float qt_coef, int qt_every,
                   int* __restrict__ status) {
    // the q and k parts of the row, then cos[rot / 2], sin[rot / 2] of the token
    extern __shared__ __align__(16) float vals[];
    __shared__ float red[66];
    // What depends on the step's metadata and on constants alone comes before the wait, while the kernel ahead ends: the
    // token's position, its cosines and sines, its page.
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    const int NQ = nq * d, NK = nkv * d, NV = nkv * dv;
    int half = rot / 2;
    float* trig = vals + NQ + NK;
    float* part = trig + rot;              // with head_norm: the sum of squares of every four neighbouring values
    float* hinv = part + (NQ + NK) / 4;    // ... and 1 / root mean square of every head
    const int pos = live ? positions[t] : 0;
    // a query's temperature: it grows with the logarithm of how many whole stretches of qt_every positions lie before it
    const float q_temp = qt_every > 0 ? 1.f + qt_coef * logf((float)((pos + 1) / qt_every) + 1.f) : 1.f;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &trig[half + i], &trig[i]);
    int page = 0;
    if (live && store_kv) {
        const int* bt = meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group];
        page = bt[pos / page_size];
        if (page <= 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
            page = 0;  // keys and values are dropped; the queries are still prepared
        }
    }
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    const TP *bias = bias_g, *q_norm = q_norm_g, *k_norm = k_norm_g;
    const float lam = (v_first && v_lambda) ? *v_lambda : 0.f;
    const size_t head_block = (size_t)page_size * dp, kv_block = (size_t)nkv * head_block;
    {
        const T* row = qkv + (size_t)t * qkv_stride;  // (the row may be the first part of a wider one)
        float sq = 0.f, sk = 0.f;
        if (vec4) {  // four values a thread (d, dv, dp and rot / 2 multiples of 4, buffers on 16 bytes)
            for (int i = threadIdx.x * 4; i < NQ + NK; i += blockDim.x * 4) {
                float v[4], bv[4] = {0.f, 0.f, 0.f, 0.f}, four = 0.f;
                load4(row + i, v);
                if (bias) load4(bias + i, bv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[k] += bv[k];
                    if (i < NQ) sq = fmaf(v[k], v[k], sq); else sk = fmaf(v[k], v[k], sk);
                    four = fmaf(v[k], v[k], four);
                }
                store4(vals + i, v);
                if (head_norm) part[i >> 2] = four;
            }
        } else {
            for (int i = threadIdx.x; i < NQ + NK; i += blockDim.x) {
                const float v = to_float(row[i]) + (bias ? to_float(bias[i]) : 0.f);
                vals[i] = v;
                if (i < NQ) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
            }
        }
        float inv_q = 1.f, inv_k = 1.f;
        if (!head_norm && (q_norm || k_norm)) {  // (its barriers also publish vals and trig)
            float both[2] = {sq, sk};
            block_sums<2>(both, red);
            if (q_norm) inv_q = rsqrtf(both[0] / (float)NQ + eps);
            if (k_norm) inv_k = rsqrtf(both[1] / (float)NK + eps);
        } else {
            __syncthreads();
        }
        const bool head_inv = head_norm && vec4;
        if (head_inv) {
            // A rotation leaves a pair's sum of squares as it is, so a head's is that of its values before the rotation:
            // a thread a head adds the fours' sums in ascending order; what follows rotates and multiplies.
            for (int h = threadIdx.x; h < nq + nkv; h += blockDim.x) {
                float ss = 0.f;
                for (int j = 0; j < d / 4; ++j) ss += part[h * (d / 4) + j];
                hinv[h] = rsqrtf(ss / (float)d + eps);
            }
            __syncthreads();
        } else if (head_norm && (q_norm || k_norm || interleaved)) {
            // a warp a head, the norm BEFORE the rotation (a weight of d elements that all heads share does not commute
            // with it): the head's sum of squares over the lanes in a fixed order, the division, the weight; what follows
            // rotates and writes the heads out
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
            for (int h = warp; h < nq + nkv; h += nwarps) {
                float* hv = vals + h * d;
                const TP* nw = h < nq ? q_norm : k_norm;
                float ss = 0.f;
                for (int i = lane; i < d; i += 32) ss = fmaf(hv[i], hv[i], ss);
                ss = warp_sum(ss);
                const float inv = rsqrtf(ss / (float)d + eps);
                __syncwarp();
                for (int i = lane; i < d; i += 32) hv[i] = hv[i] * inv * (nw ? to_float(nw[i]) : 1.f);
            }
            __syncthreads();
            q_norm = k_norm = nullptr;
        } else if (head_norm) {
            // a warp a head: the rotation in place, the head's sum of squares over the lanes in a fixed order, the division;
            // what follows writes the heads out as they are
            const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
            for (int h = warp; h < nq + nkv; h += nwarps) {
                float* hv = vals + h * d;
                float ss = 0.f;
                for (int i = lane; i < half; i += 32) {
                    float lo, hi;
                    rotate_pair(hv[i], hv[i + half], trig[i], trig[half + i], lo, hi);
                    hv[i] = lo;
                    hv[i + half] = hi;
                    ss = fmaf(lo, lo, ss);
                    ss = fmaf(hi, hi, ss);
                }
                for (int i = rot + lane; i < d; i += 32) ss = fmaf(hv[i], hv[i], ss);
                ss = warp_sum(ss);
                const float inv = rsqrtf(ss / (float)d + eps);
                __syncwarp();
                for (int i = lane; i < d; i += 32) hv[i] *= inv;
            }
            __syncthreads();
            half = 0;
            rot = 0;
        }
        const int slot = pos % page_size;
        T* kpage = cache + (size_t)page * 2 * kv_block + (size_t)slot * dp;
        T* vpage = kpage + kv_block;
        const int heads = nq + (page > 0 ? nkv : 0);
        if (vec4) {
            // q and k: one item per (head, four dims); an item of the rotated part's first half also makes its partner, so a
            // head has dp / 4 - half / 4 items.  Head and item of a thread move on by additions (no division in the loop).
            const int halfv = interleaved ? 0 : half;  // (interleaved pairs lie inside an item: no partner item)
            const int upd = dp / 4, hq = halfv / 4, uh = upd - hq;
            {
                int h = threadIdx.x / uh, u = threadIdx.x % uh;
                const int dh = blockDim.x / uh, du = blockDim.x % uh;
                while (h < heads) {
                    const int i = u < hq ? 4 * u : 4 * u + halfv;
                    const bool is_q = h < nq;
                    T* dst = is_q ? q_out + ((size_t)t * nq + h) * dp : kpage + (size_t)(h - nq) * head_block;
                    // k heads follow the q heads in vals; a weight beside a norm per head has d elements, for every head
                    const int base = h * d, nb = head_inv ? 0 : (is_q ? base : base - NQ);
                    const float inv = (head_inv ? hinv[h] : (is_q ? inv_q : inv_k)) * (is_q ? q_temp : 1.f);
                    const TP* nw = is_q ? q_norm : k_norm;
                    auto normed4 = [&](int j, float (&o)[4]) {
                        float wv[4] = {1.f, 1.f, 1.f, 1.f};
                        load4(vals + base + j, o);
                        if (nw) load4(nw + nb + j, wv);
#pragma unroll
                        for (int k = 0; k < 4; ++k) o[k] = o[k] * inv * wv[k];
                    };
                    float r[4] = {0.f, 0.f, 0.f, 0.f};
                    if (u < hq) {
                        float a[4], b[4], hi[4], cs[4], sn[4];
                        normed4(i, a);
                        normed4(i + half, b);
                        load4(trig + i, cs);
                        load4(trig + half + i, sn);
#pragma unroll
                        for (int k = 0; k < 4; ++k) rotate_pair(a[k], b[k], cs[k], sn[k], r[k], hi[k]);
                        store4(dst + i + half, hi);
                    } else if (i < d) {
                        normed4(i, r);
                        if (interleaved && i < rot) {  // dimension 2j with 2j + 1, both inside this item
                            const float a0 = r[0], b0 = r[1], a1 = r[2], b1 = r[3];
                            rotate_pair(a0, b0, trig[i / 2], trig[half + i / 2], r[0], r[1]);
                            rotate_pair(a1, b1, trig[i / 2 + 1], trig[half + i / 2 + 1], r[2], r[3]);
                        }
                    }
                    store4(dst + i, r);
                    u += du;
                    h += dh;
                    if (u >= uh) { u -= uh; ++h; }
                }
            }
            if (page > 0 || v_out) {
                int h = threadIdx.x / upd, u = threadIdx.x % upd;
                const int dh = blockDim.x / upd, du = blockDim.x % upd;
                while (h < nkv) {
                    const int i = 4 * u;
                    float r[4] = {0.f, 0.f, 0.f, 0.f};
                    if (i < dv) {
                        const int j = h * dv + i;
                        float bv[4] = {0.f, 0.f, 0.f, 0.f};
                        load4(row + NQ + NK + j, r);
                        if (bias) load4(bias + NQ + NK + j, bv);
#pragma unroll
                        for (int k = 0; k < 4; ++k) r[k] += bv[k];
                        if (v_out) store4(v_out + (size_t)t * NV + j, r);
                        if (v_first) {
                            float f[4];
                            load4(v_first + (size_t)t * NV + j, f);
#pragma unroll
                            for (int k = 0; k < 4; ++k) r[k] = (1.f - lam) * r[k] + lam * f[k];
                        }
                    }
                    if (page > 0) store4(vpage + (size_t)h * head_block + i, r);
                    u += du;
                    h += dh;
                    if (u >= upd) { u -= upd; ++h; }
                }
            }
            return;
        }
        // q and k: one item per (head, dim below dp); pairs of the rotated part are computed twice, once per half
        for (int it = threadIdx.x; it < heads * dp; it += blockDim.x) {
            const int h = it / dp, i = it % dp;
            const bool is_q = h < nq;
            T* dst = is_q ? q_out + ((size_t)t * nq + h) * dp : kpage + (size_t)(h - nq) * head_block;
            float r = 0.f;
            if (i < d) {
                const int base = h * d;
                const float inv = is_q ? inv_q : inv_k;
                const TP* nw = is_q ? q_norm : k_norm;
                const int nb = is_q ? base : base - NQ;
                auto normed = [&](int j) { return vals[base + j] * inv * (nw ? to_float(nw[nb + j]) : 1.f); };
                if (i < rot && interleaved) {
                    const int f = i >> 1;
                    float lo, hi;
                    rotate_pair(normed(i & ~1), normed(i | 1), trig[f], trig[half + f], lo, hi);
                    r = i & 1 ? hi : lo;
                } else if (i < rot) {
                    const int f = i < half ? i : i - half;
                    float lo, hi;
                    rotate_pair(normed(f), normed(f + half), trig[f], trig[half + f], lo, hi);
                    r = i < half ? lo : hi;
                } else {
                    r = normed(i);
                }
                if (is_q) r *= q_temp;
            }
            dst[i] = from_float<T>(r);
        }
        for (int it = threadIdx.x; it < nkv * dp; it += blockDim.x) {
            const int h = it / dp, i = it % dp;
            float r = 0.f;
            if (i < dv) {
                const int j = h * dv + i;
                r = to_float(row[NQ + NK + j]) + (bias ? to_float(bias[NQ + NK + j]) : 0.f);
                if (v_out) v_out[(size_t)t * NV + j] = from_float<T>(r);
                if (v_first) r = (1.f - lam) * r + lam * to_float(v_first[(size_t)t * NV + j]);
            }
            if (page > 0) vpage[(size_t)h * head_block + i] = from_float<T>(r);
        }
    }
}

// param_dtype: the type of bias, q_norm and k_norm (bfloat16 weights of a checkpoint may stay as they are stored: the
// kernel widens them, exactly, as it reads them, and a token's row then brings half as many weight bytes with it)
extern "C" int qkv_prepare(const void* qkv, long long qkv_stride, int dtype, const void* bias, const void* q_norm, const void* k_norm, int param_dtype, float eps,
                           const int* positions, const int* token_entry, const int* meta, int group, const float* inv_freq,
                           int rot, const void* v_first, const float* v_lambda, void* v_out, void* q_out, void* cache, int T,
                           int nq, int nkv, int d, int dv, int dp, int page_size, int num_pages, int store_kv, int head_norm,
                           int interleaved, float qt_coef, int qt_every, int* status, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (interleaved && rot % 2) return (int)cudaErrorInvalidValue;
    const size_t smem = ((size_t)(nq + nkv) * d + rot + (head_norm ? (size_t)(nq + nkv) * (d / 4 + 1) : 0)) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    // Few tokens: 256 threads a block, the shortest path through a token.  Many: 128, so that more blocks, each at another
    // of its phases, share a multiprocessor (16,384 tokens of 32 + 8 heads of 64: 143 -> 107 us).
    const int threads = (nq + nkv) * d >= 1024 && T < 512 ? 256 : 128;
    const uintptr_t all = (uintptr_t)qkv | (uintptr_t)bias | (uintptr_t)q_norm | (uintptr_t)k_norm | (uintptr_t)v_first |
                          (uintptr_t)v_out | (uintptr_t)q_out | (uintptr_t)cache;
    const int vec4 = d % 4 == 0 && dv % 4 == 0 && dp % 4 == 0 && rot % (interleaved ? 4 : 8) == 0 && qkv_stride % 4 == 0 && (all & 15) == 0;
    cudaError_t e;
    static size_t configured[3] = {0, 0, 0};  // the attribute only ever grows (and is not set inside a capture again)
#define PREP_CASE(TT, TP, which) \
    do { \
        if (smem > 48 * 1024 && smem > configured[which]) { \
            e = cudaFuncSetAttribute(qkv_prepare_kernel<TT, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
            configured[which] = smem; \
        } \
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, qkv_prepare_kernel<TT, TP>, T, threads, smem, stream, \
                                      (const TT*)qkv, qkv_stride, (const TP*)bias, (const TP*)q_norm, (const TP*)k_norm, eps, positions, token_entry, meta, group, inv_freq, rot, \
                                      (const TT*)v_first, v_lambda, (TT*)v_out, (TT*)q_out, (TT*)cache, nq, nkv, d, dv, dp, \
                                      page_size, num_pages, store_kv, vec4, head_norm, interleaved, qt_coef, qt_every, status); \
    } while (0)
    if (dtype == DT_F32 && param_dtype != DT_F32) return (int)cudaErrorInvalidValue;
    if (dtype == DT_F32) PREP_CASE(float, float, 0);
    if (param_dtype == DT_F32) PREP_CASE(__nv_bfloat16, float, 1);
    PREP_CASE(__nv_bfloat16, __nv_bfloat16, 2);
#undef PREP_CASE
}

// ----------------------------------------------------------------------------- polynomial activation of normalised powers
// out[t] = a N(z) + b N(z^2) + c N(z^3) + e with N(u) = u / sqrt(mean(u^2) + eps) over the row; powers element by
// element; coef = (a, b, c, e).  The three mean squares are sums of z^2, z^4 and z^6, taken in one pass.
template <typename T, int PER_THREAD>
__global__ void __launch_bounds__(1024)
polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps, T* __restrict__ out,
                const int* __restrict__ meta, int F, int wide) {
    __shared__ float red[99];
    // Up to PER_THREAD (16 or 32) values a thread stay in registers between the two passes, as they were loaded (16
    // bytes a load: a bfloat16 row costs half the registers of a float32 one, which lets more warps share a multiprocessor).
    constexpr int VEC = 16 / sizeof(T), MAXC = PER_THREAD / VEC;
    const float a = coef[0], b = coef[1], c = coef[2], e0 = coef[3];
    const int t = blockIdx.x;
    const bool live = !meta || t < meta[META_NUM_TOKENS];  // (metadata and coefficients: read before the wait)
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    const T* zr = z + (size_t)t * F;
    T* o = out + (size_t)t * F;
    float s2 = 0.f, s4 = 0.f, s6 = 0.f;
    const bool in_regs = wide && F <= VEC * MAXC * (int)blockDim.x;
    uint4 raw[MAXC];
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < MAXC; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * VEC;
            if (i < F) raw[j] = *reinterpret_cast<const uint4*>(zr + i);
        }
#pragma unroll
        for (int j = 0; j < MAXC; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * VEC;
            if (i < F) {
                const T* e = reinterpret_cast<const T*>(&raw[j]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float x = to_float(e[k]), x2 = x * x, x3 = x2 * x;
                    s2 += x2;
                    s4 = fmaf(x2, x2, s4);
                    s6 = fmaf(x3, x3, s6);
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x) {
            const float x = to_float(zr[i]), x2 = x * x, x3 = x2 * x;
            s2 += x2;
            s4 = fmaf(x2, x2, s4);
            s6 = fmaf(x3, x3, s6);
        }
    }
    float sums[3] = {s2, s4, s6};
    block_sums<3>(sums, red);
    const float n1 = a * rsqrtf(sums[0] / (float)F + eps), n2 = b * rsqrtf(sums[1] / (float)F + eps),
                n3 = c * rsqrtf(sums[2] / (float)F + eps);
    if (in_regs) {
        // the values are unpacked again from what was loaded: held unpacked since the first pass they would cost twice
        // the registers (the empty statement keeps the compiler from doing just that)
#pragma unroll
        for (int j = 0; j < MAXC; ++j) asm volatile("" : "+r"(raw[j].x), "+r"(raw[j].y), "+r"(raw[j].z), "+r"(raw[j].w));
#pragma unroll
        for (int j = 0; j < MAXC; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * VEC;
            if (i < F) {
                const T* e = reinterpret_cast<const T*>(&raw[j]);
                uint4 res;
                T* r = reinterpret_cast<T*>(&res);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const float x = to_float(e[k]), x2 = x * x;
                    r[k] = from_float<T>(n1 * x + n2 * x2 + n3 * (x2 * x) + e0);
                }
                *reinterpret_cast<uint4*>(o + i) = res;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float x = to_float(zr[i]), x2 = x * x;
        o[i] = from_float<T>(n1 * x + n2 * x2 + n3 * (x2 * x) + e0);
    }
}

extern "C" int polynorm(const void* z, int dtype, const float* coef, float eps, void* out, const int* meta, int T, int F,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    // rows of whole 16-byte pieces that start on 16 bytes
    const int wide = F % (dtype == DT_F32 ? 4 : 8) == 0 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0;
    // as many threads as keep a row in registers, 16 values each (32 for rows beyond 16,384 values), 128 at least and
    // 1024 at most
    const int per = F <= 16 * 1024 ? 16 : 32;
    int threads = ((F + per - 1) / per + 31) / 32 * 32;
    threads = threads < 128 ? 128 : threads > 1024 ? 1024 : threads;
#define POLY_CASE(TT, PER) \
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, polynorm_kernel<TT, PER>, T, threads, 0, stream, (const TT*)z, coef, eps, \
                                  (TT*)out, meta, F, wide)
    if (dtype == DT_F32) {
        if (per == 16) POLY_CASE(float, 16);
        POLY_CASE(float, 32);
    }
    if (per == 16) POLY_CASE(__nv_bfloat16, 16);
    POLY_CASE(__nv_bfloat16, 32);
#undef POLY_CASE
}
