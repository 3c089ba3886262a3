// Kernels around the residual stream of blocks whose sublayers run side by side: the pending sum of several
// terms (with a factor, rows of another stream and a vector) taken in float32 together with the norm that follows,
// and elementwise activations.  float32 and bfloat16 storage alike; all arithmetic is float32, and every reduction
// runs in an order that depends only on the row it belongs to.
#include "common.cuh"

int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

// resid[t] <- resid[t] + mult * (f0 a0[t] + f1 a1[t] + ...) + add_rows[t] + vec, up to four terms, each of the terms,
// add_rows, vec optional; out[t] = resid[t] * rsqrt(mean(resid[t]^2) + eps) * w if `out` is given, and out2 likewise with
// w2 and eps2 (two sublayers that read the same stream through norms of their own).  With `rows`: works on rows[r] of the
// inputs, writes out[r], leaves resid untouched.  The updated row waits in shared memory between the two passes.
#define SUM_MAX_TERMS 4
struct SumTerms {
    const void* p[SUM_MAX_TERMS];
    float f[SUM_MAX_TERMS];
    int n;
};

template <typename TD, typename TO>
__global__ void __launch_bounds__(256)
sum_rmsnorm_kernel(float* __restrict__ resid, SumTerms terms, float mult, const float* __restrict__ add_rows,
                   const float* __restrict__ vec, const int* __restrict__ rows, const float* __restrict__ w, float eps,
                   TO* __restrict__ out, const float* __restrict__ w2, float eps2, TO* __restrict__ out2,
                   const int* __restrict__ meta, int H, int vec4) {
    __shared__ float red[33];
    extern __shared__ __align__(16) float row[];
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int limit = rows ? meta[META_NUM_ROWS] : meta[META_NUM_TOKENS];
    if (r >= limit) return;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* x = resid + src * H;
    const TD* pt[SUM_MAX_TERMS];
#pragma unroll
    for (int j = 0; j < SUM_MAX_TERMS; ++j) pt[j] = j < terms.n ? (const TD*)terms.p[j] + src * H : nullptr;
    const float* pr = add_rows ? add_rows + src * H : nullptr;
    float ss = 0.f;
    if (vec4) {  // four values a thread and step, 16-byte accesses; the sum's order differs from the scalar form's, but is as fixed
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4];
            load4(x + i, v);
            if (terms.n > 0) {
                float s[4];
                load4(pt[0] + i, s);
                if (terms.f[0] != 1.f) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) s[k] *= terms.f[0];
                }
#pragma unroll
                for (int j = 1; j < SUM_MAX_TERMS; ++j) {
                    if (j < terms.n) {
                        float t[4];
                        load4(pt[j] + i, t);
#pragma unroll
                        for (int k = 0; k < 4; ++k) s[k] = fmaf(terms.f[j], t[k], s[k]);
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] = fmaf(mult, s[k], v[k]);
            }
            if (pr) {
                float t[4];
                load4(pr + i, t);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += t[k];
            }
            if (vec) {
                float t[4];
                load4(vec + i, t);
#pragma unroll
                for (int k = 0; k < 4; ++k) v[k] += t[k];
            }
            if (!rows) store4(x + i, v);
            store4(row + i, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(v[k], v[k], ss);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = x[i];
            if (terms.n > 0) {
                float s = to_float(pt[0][i]);
                if (terms.f[0] != 1.f) s *= terms.f[0];
#pragma unroll
                for (int j = 1; j < SUM_MAX_TERMS; ++j)
                    if (j < terms.n) s = fmaf(terms.f[j], to_float(pt[j][i]), s);
                v = fmaf(mult, s, v);
            }
            if (pr) v += pr[i];
            if (vec) v += vec[i];
            if (!rows) x[i] = v;
            row[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    if (!out) return;
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps), inv2 = rsqrtf(ss / (float)H + eps2);
    TO* o = out + (size_t)r * H;
    TO* o2 = out2 ? out2 + (size_t)r * H : nullptr;
    if (vec4) {
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float v[4], wv[4], u[4];
            load4(row + i, v);
            load4(w + i, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) u[k] = v[k] * inv * wv[k];
            store4(o + i, u);
            if (o2) {
                load4(w2 + i, wv);
#pragma unroll
                for (int k = 0; k < 4; ++k) u[k] = v[k] * inv2 * wv[k];
                store4(o2 + i, u);
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        o[i] = from_float<TO>(row[i] * inv * w[i]);
        if (o2) o2[i] = from_float<TO>(row[i] * inv2 * w2[i]);
    }
}

extern "C" int sum_rmsnorm_terms(float* resid, int num_terms, const void* const* term_ptrs, const float* factors, int term_dtype,
                                 float mult, const float* add_rows, const float* vec, const int* rows, const float* w, float eps,
                                 void* out, const float* w2, float eps2, void* out2, int out_dtype, const int* meta, int n, int H,
                                 cudaStream_t stream) {
    if (n <= 0) return 0;
    if (num_terms < 0 || num_terms > SUM_MAX_TERMS) return (int)cudaErrorInvalidValue;
    SumTerms terms = {};
    terms.n = num_terms;
    uintptr_t all = (uintptr_t)resid | (uintptr_t)add_rows | (uintptr_t)vec | (uintptr_t)w | (uintptr_t)out | (uintptr_t)w2 | (uintptr_t)out2;
    for (int j = 0; j < num_terms; ++j) {
        terms.p[j] = term_ptrs[j];
        terms.f[j] = factors ? factors[j] : 1.f;
        all |= (uintptr_t)term_ptrs[j];
    }
    const int threads = H >= 1024 ? 256 : 128;
    const size_t smem = (size_t)H * sizeof(float);
    // four values per access: rows start on multiples of four elements and the buffers on 16 bytes
    const int vec4 = H % 4 == 0 && (all & 15) == 0;
#define SUM_CASE(TD, TO)                                                                                                  \
    do {                                                                                                                  \
        static size_t configured = 0;                                                                                     \
        if (smem > 48 * 1024 && smem > configured) {                                                                      \
            cudaError_t e = cudaFuncSetAttribute(sum_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                                          \
            configured = smem;                                                                                            \
        }                                                                                                                 \
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, sum_rmsnorm_kernel<TD, TO>, n, threads, smem, stream, resid,  \
                                      terms, mult, add_rows, vec, rows, w, eps, (TO*)out, w2, eps2, (TO*)out2, meta, H, vec4); \
    } while (0)
    if (term_dtype == DT_F32 && out_dtype == DT_F32) SUM_CASE(float, float);
    else if (term_dtype == DT_BF16 && out_dtype == DT_BF16) SUM_CASE(__nv_bfloat16, __nv_bfloat16);
    else if (term_dtype == DT_F32 && out_dtype == DT_BF16) SUM_CASE(float, __nv_bfloat16);
    else SUM_CASE(__nv_bfloat16, float);
#undef SUM_CASE
}

extern "C" int sum_rmsnorm(float* resid, const void* a, const void* b, int term_dtype, float mult, const float* add_rows,
                           const float* vec, const int* rows, const float* w, float eps, void* out, int out_dtype,
                           const int* meta, int n, int H, cudaStream_t stream) {
    const void* ptrs[2] = {a, b};
    return sum_rmsnorm_terms(resid, a ? (b ? 2 : 1) : 0, ptrs, nullptr, term_dtype, mult, add_rows, vec, rows, w, eps, out, nullptr,
                             0.f, nullptr, out_dtype, meta, n, H, stream);
}

// ----------------------------------------------------------------------------- elementwise activations
// kind 0: the tanh form of GELU, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); kind 1: the square of relu, max(z, 0)^2.
__device__ __forceinline__ float gelu_tanh(float z) {
    // 0.5 (1 + tanh u) = 1 / (1 + exp(-2u))
    const float u = 0.7978845608028654f * fmaf(0.044715f * z * z, z, z);
    return z / (1.f + expf(-2.f * u));
}

__device__ __forceinline__ float relu_squared(float z) {
    const float r = fmaxf(z, 0.f);
    return r * r;
}
__device__ __forceinline__ float activate(float z, int kind) { return kind == 1 ? relu_squared(z) : gelu_tanh(z); }

template <typename T>
__global__ void __launch_bounds__(256)
activation_kernel(const T* __restrict__ z, T* __restrict__ out, const int* __restrict__ meta, int n, int kind, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int V = 16 / sizeof(T);  // elements of a 16-byte access
    const size_t total = (size_t)meta[META_NUM_TOKENS] * n;
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (i >= total) return;
    if (vec && i + V <= total) {
        float v[V];
#pragma unroll
        for (int k = 0; k < V; k += 4) {
            float t4[4];
            load4(z + i + k, t4);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[k + j] = activate(t4[j], kind);
        }
#pragma unroll
        for (int k = 0; k < V; k += 4) {
            const float o4[4] = {v[k], v[k + 1], v[k + 2], v[k + 3]};
            store4(out + i + k, o4);
        }
        return;
    }
    for (size_t k = i; k < total && k < i + V; ++k) out[k] = from_float<T>(activate(to_float(z[k]), kind));
}

extern "C" int activation_rows(const void* z, void* out, int dtype, const int* meta, int T, int n, int kind,
                               cudaStream_t stream) {
    if (T <= 0 || n <= 0) return 0;
    if (kind != 0 && kind != 1) return (int)cudaErrorInvalidValue;
    const int V = dtype == DT_F32 ? 4 : 8;
    const size_t total = (size_t)T * n;
    const unsigned blocks = (unsigned)((total + 256 * V - 1) / (256 * V));
    const int vec = (((uintptr_t)z | (uintptr_t)out) & 15) == 0;  // (rows are contiguous: element i of the whole lies at i)
    if (dtype == DT_F32)
        return (int)launch_kernel(activation_kernel<float>, blocks, 256, 0, stream, (const float*)z, (float*)out, meta, n, kind, vec);
    return (int)launch_kernel(activation_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)z,
                              (__nv_bfloat16*)out, meta, n, kind, vec);
}
