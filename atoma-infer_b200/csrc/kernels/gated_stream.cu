// Kernels of blocks that norm a sublayer's input AND its result, let the mixer read its input shifted toward the token
// before, and gate every result by a sigmoid of the sublayer's input; plus the small maps such layers bring along (a
// clamped gated activation, a gate per head, a norm over the whole row with a gate, a scaled soft cap).  float32 and
// bfloat16 storage alike; all arithmetic is float32, and every reduction runs in an order that depends only on the row.
#include "common.cuh"

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// `scratch` holds 66 floats.  Two block sums at once, each in the order of block_sum.
__device__ __forceinline__ void block_sum_pair(float& a, float& b, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();
    if (lane == 0) { scratch[warp] = a; scratch[33 + warp] = b; }
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f, u = lane < nwarps ? scratch[33 + lane] : 0.f;
        t = warp_sum(t);
        u = warp_sum(u);
        if (lane == 0) { scratch[32] = t; scratch[65] = u; }
    }
    __syncthreads();
    a = scratch[32];
    b = scratch[65];
}

// ----------------------------------------------------------------------------- norm, and the row shifted toward the row before
// h[t] = resid[t] * rsqrt(mean(resid[t]^2) + eps) * w;  hs[t] = h[t] + (h[t - 1] - h[t]) * mu, where h[t - 1] is the normed
// row of the token before in the same request: recomputed here from resid[t - 1] if that token is in this step (the
// same arithmetic, so the same bits as its own block gets), else the request's kept row `state[slot]`, else (position 0)
// zeros.  The last row of every entry goes to `last[entry]`; the kernel that ends the sublayer moves it into the state
// (this kernel's other blocks may still be reading the old one).  `h` and/or `hs` may be null.
template <typename TO>
__global__ void __launch_bounds__(256)
norm_shift_kernel(const float* __restrict__ resid, const float* __restrict__ w, float eps, const float* __restrict__ mu,
                  const float* __restrict__ state, long long slot_stride, TO* __restrict__ h, TO* __restrict__ hs,
                  float* __restrict__ last, const int* __restrict__ meta, const int* __restrict__ positions,
                  const int* __restrict__ token_entry, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int H,
                  int vec4) {
    __shared__ float red[66];
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    int e = 0, first = 0, end = 0, pos = 0, slot = 0;
    if (live) {
        e = token_entry[t];
        first = cu_tokens[e];
        end = cu_tokens[e + 1];
        pos = positions[t];
        slot = slots[e];
    }
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    const float* x = resid + (size_t)t * H;
    const bool from_row = mu && t > first, from_state = mu && !from_row && pos > 0 && state;
    const float* xp = from_row ? x - H : nullptr;
    const float* sp = from_state ? state + (size_t)slot * slot_stride : nullptr;
    float ss = 0.f, sp2 = 0.f;
    if (vec4) {  // four values a thread and step, 16-byte accesses; the sums' order differs from the scalar form's, but is as fixed
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4];
            load4(x + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(v[k], v[k], ss);
            if (from_row) {
                load4(xp + i, v);
#pragma unroll
                for (int k = 0; k < 4; ++k) sp2 = fmaf(v[k], v[k], sp2);
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = x[i];
            ss = fmaf(v, v, ss);
            if (from_row) { const float u = xp[i]; sp2 = fmaf(u, u, sp2); }
        }
    }
    block_sum_pair(ss, sp2, red);
    const float inv = rsqrtf(ss / (float)H + eps), invp = rsqrtf(sp2 / (float)H + eps);
    const bool keep = last && t == end - 1;
    if (vec4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4], wv[4], hv[4];
            load4(x + i, v);
            load4(w + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) hv[k] = v[k] * inv * wv[k];
            if (h) store4(h + (size_t)t * H + i, hv);
            if (keep) store4(last + (size_t)e * H + i, hv);
            if (hs) {
                float before[4] = {0.f, 0.f, 0.f, 0.f}, o[4];
                if (from_row) {
                    load4(xp + i, before);
#pragma unroll
                    for (int k = 0; k < 4; ++k) before[k] = before[k] * invp * wv[k];
                } else if (from_state) {
                    load4(sp + i, before);
                }
                if (mu) {
                    float m4[4];
                    load4(mu + i, m4);
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = hv[k] + (before[k] - hv[k]) * m4[k];
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k) o[k] = hv[k];
                }
                store4(hs + (size_t)t * H + i, o);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float hv = x[i] * inv * w[i];
        if (h) h[(size_t)t * H + i] = from_float<TO>(hv);
        if (keep) last[(size_t)e * H + i] = hv;
        if (hs) {
            float before = 0.f;
            if (from_row) before = xp[i] * invp * w[i];
            else if (from_state) before = sp[i];
            hs[(size_t)t * H + i] = from_float<TO>(mu ? hv + (before - hv) * mu[i] : hv);
        }
    }
}

extern "C" int norm_shift(const float* resid, const float* w, float eps, const float* mu, const float* state, long long slot_stride,
                          void* h, void* hs, int out_dtype, float* last, const int* meta, const int* positions,
                          const int* token_entry, const int* cu_tokens, const int* slots, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    // four values per access: rows start on multiples of four elements and the buffers on 16 bytes
    const uintptr_t all = (uintptr_t)resid | (uintptr_t)w | (uintptr_t)mu | (uintptr_t)state | (uintptr_t)h | (uintptr_t)hs | (uintptr_t)last;
    const int vec4 = H % 4 == 0 && slot_stride % 4 == 0 && (all & 15) == 0;
    if (out_dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, norm_shift_kernel<float>, T, threads, 0, stream, resid, w, eps, mu, state,
                                      slot_stride, (float*)h, (float*)hs, last, meta, positions, token_entry, cu_tokens, slots, H, vec4);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, norm_shift_kernel<__nv_bfloat16>, T, threads, 0, stream, resid, w, eps, mu,
                                  state, slot_stride, (__nv_bfloat16*)h, (__nv_bfloat16*)hs, last, meta, positions, token_entry,
                                  cu_tokens, slots, H, vec4);
}

// ----------------------------------------------------------------------------- gate, norm of the result, sum into the stream
// y = mult * (f0 a0[t] + f1 a1[t] + ...) + vec;  y *= sigmoid(gate[t] + gate_bias);  resid[t] += y * rsqrt(mean(y^2) + eps) * w.
// With `w_next`: also out[t] = resid[t] * rsqrt(mean(resid[t]^2) + eps_next) * w_next, the next sublayer's input.
// With `last` and `state`: the block of an entry's last row moves last[entry] into state[slot] (the row kept for the next
// step's shift; see norm_shift).
#define GATED_MAX_TERMS 4
struct GatedTerms {
    const void* p[GATED_MAX_TERMS];
    float f[GATED_MAX_TERMS];
    int n;
};

template <typename TD, typename TG, typename TO>
__global__ void __launch_bounds__(256)
gated_norm_add_kernel(float* __restrict__ resid, GatedTerms terms, float mult, const float* __restrict__ vec,
                      const TG* __restrict__ gate, const float* __restrict__ gate_bias, const float* __restrict__ w, float eps,
                      const float* __restrict__ w_next, float eps_next, TO* __restrict__ out, const float* __restrict__ last,
                      float* __restrict__ state, long long slot_stride, const int* __restrict__ meta,
                      const int* __restrict__ token_entry, const int* __restrict__ cu_tokens, const int* __restrict__ slots, int H,
                      int vec4) {
    __shared__ float red[33];
    extern __shared__ __align__(16) float row[];
    const int t = blockIdx.x;
    const bool live = t < meta[META_NUM_TOKENS];
    int e = 0, end = 0, slot = 0;
    if (live && last) {
        e = token_entry[t];
        end = cu_tokens[e + 1];
        slot = slots[e];
    }
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    if (last && t == end - 1) {
        float* dst = state + (size_t)slot * slot_stride;
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = last[(size_t)e * H + i];
    }
    float ss = 0.f;
    if (vec4) {  // four values a thread and step, 16-byte accesses; the sums' order differs from the scalar form's, but is as fixed
        float* x = resid + (size_t)t * H;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            if (terms.n > 0) {
                load4((const TD*)terms.p[0] + (size_t)t * H + i, s);
                if (terms.f[0] != 1.f) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) s[k] *= terms.f[0];
                }
#pragma unroll
                for (int j = 1; j < GATED_MAX_TERMS; ++j) {
                    if (j < terms.n) {
                        float u[4];
                        load4((const TD*)terms.p[j] + (size_t)t * H + i, u);
#pragma unroll
                        for (int k = 0; k < 4; ++k) s[k] = fmaf(terms.f[j], u[k], s[k]);
                    }
                }
                if (mult != 1.f) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) s[k] *= mult;
                }
            }
            if (vec) {
                float u[4];
                load4(vec + i, u);
#pragma unroll
                for (int k = 0; k < 4; ++k) s[k] += u[k];
            }
            if (gate) {
                float gv[4], gb[4] = {0.f, 0.f, 0.f, 0.f};
                load4(gate + (size_t)t * H + i, gv);
                if (gate_bias) load4(gate_bias + i, gb);
#pragma unroll
                for (int k = 0; k < 4; ++k) s[k] *= sigmoid_f(gv[k] + gb[k]);
            }
            store4(row + i, s);
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(s[k], s[k], ss);
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)H + eps);
        float s2 = 0.f;
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4], r[4], wv[4];
            load4(x + i, v);
            load4(row + i, r);
            load4(w + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                v[k] += r[k] * inv * wv[k];
                s2 = fmaf(v[k], v[k], s2);
            }
            store4(x + i, v);
            store4(row + i, v);
        }
        if (!w_next) return;
        s2 = block_sum(s2, red);
        const float inv2 = rsqrtf(s2 / (float)H + eps_next);
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4], wv[4];
            load4(row + i, v);
            load4(w_next + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = v[k] * inv2 * wv[k];
            store4(out + (size_t)t * H + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float s = 0.f;
        if (terms.n > 0) {
            s = to_float(((const TD*)terms.p[0])[(size_t)t * H + i]);
            if (terms.f[0] != 1.f) s *= terms.f[0];
#pragma unroll
            for (int j = 1; j < GATED_MAX_TERMS; ++j)
                if (j < terms.n) s = fmaf(terms.f[j], to_float(((const TD*)terms.p[j])[(size_t)t * H + i]), s);
            if (mult != 1.f) s *= mult;
        }
        if (vec) s += vec[i];
        if (gate) s *= sigmoid_f(to_float(gate[(size_t)t * H + i]) + (gate_bias ? gate_bias[i] : 0.f));
        row[i] = s;
        ss = fmaf(s, s, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    float* x = resid + (size_t)t * H;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = x[i] + row[i] * inv * w[i];
        x[i] = v;
        row[i] = v;
        s2 = fmaf(v, v, s2);
    }
    if (!w_next) return;
    s2 = block_sum(s2, red);
    const float inv2 = rsqrtf(s2 / (float)H + eps_next);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = from_float<TO>(row[i] * inv2 * w_next[i]);
}

extern "C" int gated_norm_add(float* resid, int num_terms, const void* const* term_ptrs, const float* factors, int term_dtype,
                              float mult, const float* vec, const void* gate, int gate_dtype, const float* gate_bias, const float* w,
                              float eps, const float* w_next, float eps_next, void* out, int out_dtype, const float* last,
                              float* state, long long slot_stride, const int* meta, const int* token_entry, const int* cu_tokens,
                              const int* slots, int T, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (num_terms < 0 || num_terms > GATED_MAX_TERMS) return (int)cudaErrorInvalidValue;
    GatedTerms terms = {};
    terms.n = num_terms;
    for (int j = 0; j < num_terms; ++j) {
        terms.p[j] = term_ptrs[j];
        terms.f[j] = factors ? factors[j] : 1.f;
    }
    const int threads = H >= 1024 ? 256 : 128;
    const size_t smem = (size_t)H * sizeof(float);
    uintptr_t all = (uintptr_t)resid | (uintptr_t)vec | (uintptr_t)gate | (uintptr_t)gate_bias | (uintptr_t)w | (uintptr_t)w_next | (uintptr_t)out;
    for (int j = 0; j < num_terms; ++j) all |= (uintptr_t)term_ptrs[j];
    const int vec4 = H % 4 == 0 && (all & 15) == 0;
#define GATED_CASE(TD, TG, TO)                                                                                             \
    do {                                                                                                                  \
        static size_t configured = 0;                                                                                     \
        if (smem > 48 * 1024 && smem > configured) {                                                                      \
            cudaError_t ce = cudaFuncSetAttribute(gated_norm_add_kernel<TD, TG, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (ce != cudaSuccess) return (int)ce;                                                                        \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, gated_norm_add_kernel<TD, TG, TO>, T, threads, smem, stream, resid, terms, \
                                      mult, vec, (const TG*)gate, gate_bias, w, eps, w_next, eps_next, (TO*)out, last, state,  \
                                      slot_stride, meta, token_entry, cu_tokens, slots, H, vec4);                          \
    } while (0)
    if (term_dtype == DT_F32) {
        if (gate_dtype != DT_F32 || out_dtype != DT_F32) return (int)cudaErrorInvalidValue;
        GATED_CASE(float, float, float);
    }
    if (out_dtype != DT_BF16) return (int)cudaErrorInvalidValue;
    if (gate_dtype == DT_F32) GATED_CASE(__nv_bfloat16, float, __nv_bfloat16);
    GATED_CASE(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
#undef GATED_CASE
}

// ----------------------------------------------------------------------------- clamped gated activation
// out[t, i] = g * sigmoid(alpha * g) * (u + 1) with g = min(gu[t, i], limit), u = clamp(gu[t, F + i], -limit, limit);
// gu is [T, 2F] (gate columns first), out [T, F].
template <typename T>
__global__ void __launch_bounds__(256)
clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, const int* __restrict__ meta, int F, float limit, float alpha,
                   int vec4) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)meta[META_NUM_TOKENS] * F;
    if (vec4) {  // four neighbouring outputs of one row a thread (F is a multiple of four)
        const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
        if (idx >= total) return;
        const size_t t = idx / F, i = idx % F;
        float g[4], u[4], o[4];
        load4(gu + t * 2 * F + i, g);
        load4(gu + t * 2 * F + F + i, u);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gg = fminf(g[k], limit), uu = fminf(fmaxf(u[k], -limit), limit);
            o[k] = gg * sigmoid_f(alpha * gg) * (uu + 1.f);
        }
        store4(out + idx, o);
        return;
    }
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / F, i = idx % F;
    const float g = fminf(to_float(gu[t * 2 * F + i]), limit);
    const float u = fminf(fmaxf(to_float(gu[t * 2 * F + F + i]), -limit), limit);
    out[idx] = from_float<T>(g * sigmoid_f(alpha * g) * (u + 1.f));
}

extern "C" int clamped_glu(const void* gu, void* out, int dtype, const int* meta, int T, int F, float limit, float alpha,
                           cudaStream_t stream) {
    if (T <= 0 || F <= 0) return 0;
    const int vec4 = F % 4 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0;
    const size_t items = vec4 ? (size_t)T * F / 4 : (size_t)T * F;
    const unsigned blocks = (unsigned)((items + 255) / 256);
    if (dtype == DT_F32)
        return (int)launch_kernel(clamped_glu_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, meta, F, limit, alpha,
                                  vec4);
    return (int)launch_kernel(clamped_glu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gu,
                              (__nv_bfloat16*)out, meta, F, limit, alpha, vec4);
}

// ----------------------------------------------------------------------------- one gate per head
// y[t, h, :] *= sigmoid(g[t, h]) in place; y [T, heads, n] with strides, g rows of g_stride elements.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ y, long long y_token, long long y_head, const T* __restrict__ g, long long g_stride,
                 const int* __restrict__ meta, int heads, int n, int vec4) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    if (vec4) {  // four neighbouring values of one head a thread and step
        const int per = n / 4;
        for (int idx = threadIdx.x; idx < heads * per; idx += blockDim.x) {
            const int hd = idx / per, i = (idx % per) * 4;
            T* p = y + (size_t)t * y_token + (size_t)hd * y_head + i;
            const float sg = sigmoid_f(to_float(g[(size_t)t * g_stride + hd]));
            float v[4];
            load4(p, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] *= sg;
            store4(p, v);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < heads * n; idx += blockDim.x) {
        const int hd = idx / n, i = idx % n;
        T* p = y + (size_t)t * y_token + (size_t)hd * y_head + i;
        *p = from_float<T>(to_float(*p) * sigmoid_f(to_float(g[(size_t)t * g_stride + hd])));
    }
}

extern "C" int head_gate(void* y, long long y_token, long long y_head, const void* g, long long g_stride, int dtype,
                         const int* meta, int T, int heads, int n, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = heads * n >= 1024 ? 256 : 128;
    const int esz = dtype == DT_F32 ? 4 : 2;
    const int vec4 = n % 4 == 0 && y_token % 4 == 0 && y_head % 4 == 0 && ((uintptr_t)y % (4 * esz)) == 0;
    if (dtype == DT_F32)
        return (int)launch_kernel(head_gate_kernel<float>, T, threads, 0, stream, (float*)y, y_token, y_head, (const float*)g,
                                  g_stride, meta, heads, n, vec4);
    return (int)launch_kernel(head_gate_kernel<__nv_bfloat16>, T, threads, 0, stream, (__nv_bfloat16*)y, y_token, y_head,
                              (const __nv_bfloat16*)g, g_stride, meta, heads, n, vec4);
}

// ----------------------------------------------------------------------------- norm over the whole row, weight, gate
// out[t] = o[t] * rsqrt(mean(o[t]^2) + eps) * w * gate(g[t]); o float32 [T, n], g a slice of wider rows, w float32 [n];
// kind 0: sigmoid(g), kind 1: g * sigmoid(g).
template <typename T>
__global__ void __launch_bounds__(256)
row_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, long long g_stride, const float* __restrict__ w,
                     float eps, T* __restrict__ out, const int* __restrict__ meta, int n, int kind, int vec4) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const float* row = o + (size_t)t * n;
    float ss = 0.f;
    if (vec4) {
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            float v[4];
            load4(row + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(v[k], v[k], ss);
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)n + eps);
        for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
            float v[4], gv[4], wv[4];
            load4(row + i, v);
            load4(g + (size_t)t * g_stride + i, gv);
            load4(w + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float sg = sigmoid_f(gv[k]);
                v[k] = v[k] * inv * wv[k] * (kind == 1 ? gv[k] * sg : sg);
            }
            store4(out + (size_t)t * n + i, v);
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float gv = to_float(g[(size_t)t * g_stride + i]), s = sigmoid_f(gv);
        out[(size_t)t * n + i] = from_float<T>(row[i] * inv * w[i] * (kind == 1 ? gv * s : s));
    }
}

extern "C" int row_norm_gate(const float* o, const void* g, int dtype, long long g_stride, const float* w, float eps, void* out,
                             const int* meta, int T, int n, int kind, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = n >= 1024 ? 256 : 128;
    const int vec4 = n % 4 == 0 && g_stride % 4 == 0 && (((uintptr_t)o | (uintptr_t)g | (uintptr_t)w | (uintptr_t)out) & 15) == 0;
    if (dtype == DT_F32)
        return (int)launch_kernel(row_norm_gate_kernel<float>, T, threads, 0, stream, o, (const float*)g, g_stride, w, eps, (float*)out,
                                  meta, n, kind, vec4);
    return (int)launch_kernel(row_norm_gate_kernel<__nv_bfloat16>, T, threads, 0, stream, o, (const __nv_bfloat16*)g, g_stride, w, eps,
                              (__nv_bfloat16*)out, meta, n, kind, vec4);
}

// ----------------------------------------------------------------------------- scaled soft cap
// z <- cap * tanh(z * scale / cap) in place (cap <= 0: z * scale); float32 [rows, n], rows from the step's metadata.
__global__ void __launch_bounds__(256)
scale_softcap_kernel(float* __restrict__ z, const int* __restrict__ meta, int n, float scale, float cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total = (size_t)meta[META_NUM_ROWS] * n;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float v = z[idx] * scale;
    z[idx] = cap > 0.f ? cap * tanhf(v / cap) : v;
}

extern "C" int scale_softcap(float* z, const int* meta, int rows, int n, float scale, float cap, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const unsigned blocks = (unsigned)(((size_t)rows * n + 255) / 256);
    return (int)launch_kernel(scale_softcap_kernel, blocks, 256, 0, stream, z, meta, n, scale, cap);
}
