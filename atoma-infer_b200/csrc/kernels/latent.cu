// Kernels of attention through low-rank latents: a root-mean-square norm over a slice of wider rows, a linear map
// applied head by head, and the rows' preparation (norm of the key/value latent, rotation of the shared key part and
// of the queries' rotated parts, the cached vector written to its page, the queries laid out for the attention
// kernels).  Storage is float32 or bfloat16, arithmetic float32.
#include <algorithm>

#include "common.cuh"

// out[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * w over n elements; x is a slice of a wider row (x_stride from row to row).
template <typename T>
__global__ void __launch_bounds__(256)
rms_rows_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ w, float eps, T* __restrict__ out,
                const int* __restrict__ meta, int n) {
    __shared__ float red[33];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const T* xr = x + (size_t)t * x_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = to_float(xr[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)t * n + i] = from_float<T>(to_float(xr[i]) * inv * w[i]);
}

extern "C" int rms_rows(const void* x, int dtype, long long x_stride, const float* w, float eps, void* out, const int* meta,
                        int T, int n, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = n >= 1024 ? 256 : 128;
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, rms_rows_kernel<float>, T, threads, 0, stream, (const float*)x, x_stride,
                                      w, eps, (float*)out, meta, n);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, rms_rows_kernel<__nv_bfloat16>, T, threads, 0, stream,
                                  (const __nv_bfloat16*)x, x_stride, w, eps, (__nv_bfloat16*)out, meta, n);
}

// ----------------------------------------------------------------------------- a linear map per head
// y[t, h, n] = sum_k x[t, h, k] * w[h, n, k] (optionally times sigmoid(gate[t, h, n])).  x, y and gate are slices:
// element (t, h, i) lies at t * stride_t + h * stride_h + i.
#define HL_TM 8
#define HL_TN 128
#define HL_KC 512
// A block takes HL_TM tokens x HL_TN outputs of one head.  The tokens' x waits in shared memory (HL_KC columns at a
// time); a thread owns one output and reads its weight row itself, 16 bytes a load where the rows allow; every output
// is one accumulator running over k in order, so its value does not depend on the tile it falls in.
template <typename T>
__global__ void __launch_bounds__(HL_TN)
head_linear_kernel(const T* __restrict__ x, long long xs_t, long long xs_h, const T* __restrict__ w, T* __restrict__ y,
                   long long ys_t, long long ys_h, const T* __restrict__ gate, long long gs_t, long long gs_h,
                   const int* __restrict__ meta, int K, int N, int wvec) {
    __shared__ float xs[HL_TM][HL_KC];
    pdl_launch_dependents();
    pdl_wait();
    const int ntok = meta[META_NUM_TOKENS];
    const int t0 = blockIdx.x * HL_TM, h = blockIdx.y, n0 = blockIdx.z * blockDim.x, tid = threadIdx.x;
    if (t0 >= ntok) return;
    const int rows = min(HL_TM, ntok - t0), n = n0 + tid;
    const T* wr = w + ((size_t)h * N + min(n, N - 1)) * K;
    constexpr int V = 16 / sizeof(T);
    float acc[HL_TM];
#pragma unroll
    for (int m = 0; m < HL_TM; ++m) acc[m] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HL_KC) {
        const int kc = min(HL_KC, K - k0);
        __syncthreads();
        for (int idx = tid; idx < HL_TM * kc; idx += blockDim.x) {
            const int m = idx / kc, kk = idx % kc;
            xs[m][kk] = m < rows ? to_float(x[(size_t)(t0 + m) * xs_t + (size_t)h * xs_h + k0 + kk]) : 0.f;
        }
        __syncthreads();
        int kk = 0;
        if (wvec) {
            for (; kk + V <= kc; kk += V) {
                const uint4 raw = *reinterpret_cast<const uint4*>(wr + k0 + kk);
                const T* wv = reinterpret_cast<const T*>(&raw);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float f = to_float(wv[i]);
#pragma unroll
                    for (int m = 0; m < HL_TM; ++m) acc[m] = fmaf(xs[m][kk + i], f, acc[m]);
                }
            }
        }
        for (; kk < kc; ++kk) {
            const float f = to_float(wr[k0 + kk]);
#pragma unroll
            for (int m = 0; m < HL_TM; ++m) acc[m] = fmaf(xs[m][kk], f, acc[m]);
        }
    }
    if (n >= N) return;
    for (int m = 0; m < rows; ++m) {
        float v = acc[m];
        if (gate) {
            const float g = to_float(gate[(size_t)(t0 + m) * gs_t + (size_t)h * gs_h + n]);
            v = v / (1.f + expf(-g));
        }
        y[(size_t)(t0 + m) * ys_t + (size_t)h * ys_h + n] = from_float<T>(v);
    }
}

extern "C" int head_linear(const void* x, long long xs_t, long long xs_h, const void* w, void* y, long long ys_t,
                           long long ys_h, const void* gate, long long gs_t, long long gs_h, int dtype, const int* meta, int T,
                           int heads, int K, int N, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int tn = N <= 32 ? 32 : (N <= 64 ? 64 : HL_TN);  // few outputs a head: smaller blocks, all of their threads at work
    dim3 grid((T + HL_TM - 1) / HL_TM, heads, (N + tn - 1) / tn);
    const int elem = dtype == DT_F32 ? 4 : 2;
    const int wvec = ((size_t)K * elem) % 16 == 0 && ((uintptr_t)w & 15) == 0;
    if (dtype == DT_F32)
        return (int)launch_kernel(head_linear_kernel<float>, grid, tn, 0, stream, (const float*)x, xs_t, xs_h, (const float*)w,
                                  (float*)y, ys_t, ys_h, (const float*)gate, gs_t, gs_h, meta, K, N, wvec);
    return (int)launch_kernel(head_linear_kernel<__nv_bfloat16>, grid, tn, 0, stream, (const __nv_bfloat16*)x, xs_t, xs_h,
                              (const __nv_bfloat16*)w, (__nv_bfloat16*)y, ys_t, ys_h, (const __nv_bfloat16*)gate, gs_t, gs_h,
                              meta, K, N, wvec);
}

// y[t, h, n] *= sigmoid(gate[t, h, n]) for a product that a library made (same slices as above).  ``vec``: every head's
// slice of y and of gate starts on 16 bytes and N is a multiple of 16 bytes' worth of elements; a thread then maps 16 bytes.
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ y, long long ys_t, long long ys_h, const T* __restrict__ gate, long long gs_t,
                    long long gs_h, const int* __restrict__ meta, int heads, int N, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    if (vec) {
        constexpr int V = 16 / (int)sizeof(T);
        for (int idx = threadIdx.x * V; idx < heads * N; idx += blockDim.x * V) {
            const int h = idx / N, n = idx % N;
            uint4 gv = *reinterpret_cast<const uint4*>(gate + (size_t)t * gs_t + (size_t)h * gs_h + n);
            uint4* at = reinterpret_cast<uint4*>(y + (size_t)t * ys_t + (size_t)h * ys_h + n);
            uint4 yv = *at;
            const T* ge = reinterpret_cast<const T*>(&gv);
            T* ye = reinterpret_cast<T*>(&yv);
#pragma unroll
            for (int i = 0; i < V; ++i) ye[i] = from_float<T>(to_float(ye[i]) / (1.f + expf(-to_float(ge[i]))));
            *at = yv;
        }
        return;
    }
    for (int idx = threadIdx.x; idx < heads * N; idx += blockDim.x) {
        const int h = idx / N, n = idx % N;
        const float g = to_float(gate[(size_t)t * gs_t + (size_t)h * gs_h + n]);
        T* at = y + (size_t)t * ys_t + (size_t)h * ys_h + n;
        *at = from_float<T>(to_float(*at) / (1.f + expf(-g)));
    }
}

extern "C" int sigmoid_gate(void* y, long long ys_t, long long ys_h, const void* gate, long long gs_t, long long gs_h,
                            int dtype, const int* meta, int T, int heads, int N, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long V = dtype == DT_F32 ? 4 : 8;
    const int vec = N % V == 0 && ys_t % V == 0 && ys_h % V == 0 && gs_t % V == 0 && gs_h % V == 0 &&
                    ((uintptr_t)y | (uintptr_t)gate) % 16 == 0;
    const int threads = (int)std::min<long long>(256, std::max<long long>(32, ((long long)heads * N / (vec ? V : 1) + 31) / 32 * 32));
    if (dtype == DT_F32)
        return (int)launch_kernel(sigmoid_gate_kernel<float>, T, threads, 0, stream, (float*)y, ys_t, ys_h, (const float*)gate, gs_t,
                                  gs_h, meta, heads, N, vec);
    return (int)launch_kernel(sigmoid_gate_kernel<__nv_bfloat16>, T, threads, 0, stream, (__nv_bfloat16*)y, ys_t, ys_h,
                              (const __nv_bfloat16*)gate, gs_t, gs_h, meta, heads, N, vec);
}

// ----------------------------------------------------------------------------- the rows of latent attention
// Per token: the cached vector [c | rotated key part | zeros] with c = dkv[:rank] * rsqrt(mean(.^2) + eps) * norm_w
// goes to the key plane and to the value plane of the token's page (one key/value head of D elements); the queries
// become [q_abs[h] | rotated q_rot[h] | zeros] of D elements a head.  Rotation: of the first `rot` dimensions of a
// rotated part, 2i pairs with 2i + 1, by the angle position * inv_freq[i] (float32 product, sincosf).
// Two neighbouring elements at once (the address a multiple of two elements): a rotation's pair.
__device__ __forceinline__ void load2(const float* p, float& a, float& b) { const float2 t = *reinterpret_cast<const float2*>(p); a = t.x; b = t.y; }
__device__ __forceinline__ void load2(const __nv_bfloat16* p, float& a, float& b) {
    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    a = t.x; b = t.y;
}
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

// A block takes one token and `hpb` of its heads + 1 jobs: job h < heads lays out query head h, job `heads` makes the
// cached vector.  Few tokens: a job a block; many: all of a token's jobs in one block, which takes the cosines and
// sines once.  `pairs`: sizes, strides and addresses are even, so a thread takes a rotation's pair with one access.
template <typename T>
__global__ void __launch_bounds__(256)
latent_rows_kernel(const T* __restrict__ q_rot, long long qs_t, long long qs_h, const T* __restrict__ q_abs,
                   const T* __restrict__ dkv, long long dkv_stride, const float* __restrict__ norm_w, float eps,
                   const int* __restrict__ positions, const int* __restrict__ token_entry, const int* __restrict__ meta,
                   int group, const float* __restrict__ inv_freq, int rot, T* __restrict__ q_out, T* __restrict__ cache,
                   int heads, int rank, int rdim, int D, int page_size, int num_pages, int store, int pairs, int hpb,
                   int* __restrict__ status) {
    __shared__ float red[33];
    extern __shared__ float cs[];  // rot / 2 cosines, rot / 2 sines
    float* sn = cs + rot / 2;
    // The step's metadata is written by no kernel of the step: it is read before the wait.
    const int t = blockIdx.x, h_first = blockIdx.y * hpb, h_end = min(heads + (store ? 1 : 0), h_first + hpb), tid = threadIdx.x;
    const bool live = t < meta[META_NUM_TOKENS] && h_first < h_end;
    const int p = live ? positions[t] : 0;
    int page = 0;
    if (live && h_end == heads + 1) page = (meta + meta[META_BT_OFFSET + group] + (size_t)token_entry[t] * meta[META_BT_STRIDE + group])[p / page_size];
    if (live)
        for (int i = tid; i < rot / 2; i += blockDim.x) sincosf((float)p * inv_freq[i], &sn[i], &cs[i]);
    pdl_wait();
    pdl_launch_dependents();
    if (!live) return;
    __syncthreads();  // the cosines and sines are written
    for (int h = h_first; h < min(h_end, heads); ++h) {
        const T* qr = q_rot + (size_t)t * qs_t + (size_t)h * qs_h;
        const T* qa = q_abs + ((size_t)t * heads + h) * rank;
        T* dst = q_out + ((size_t)t * heads + h) * D;
        if (pairs) {
            for (int i = tid * 2; i < D; i += blockDim.x * 2) {
                float a = 0.f, b = 0.f;
                if (i < rank) {
                    load2(qa + i, a, b);
                } else if (i < rank + rdim) {
                    const int j = i - rank;
                    load2(qr + j, a, b);
                    if (j < rot) {
                        const float a0 = a, b0 = b;
                        rotate_pair(a0, b0, cs[j >> 1], sn[j >> 1], a, b);
                    }
                }
                store2(dst + i, a, b);
            }
            continue;
        }
        for (int i = tid; i < D; i += blockDim.x) {
            float v = 0.f;
            if (i < rank) {
                v = to_float(qa[i]);
            } else if (i < rank + rdim) {
                const int j = i - rank;
                v = to_float(qr[j]);
                if (j < rot) {
                    const float other = to_float(qr[j ^ 1]);
                    float lo, hi;
                    if (j & 1) { rotate_pair(other, v, cs[j >> 1], sn[j >> 1], lo, hi); v = hi; }
                    else { rotate_pair(v, other, cs[j >> 1], sn[j >> 1], lo, hi); v = lo; }
                }
            }
            dst[i] = from_float<T>(v);
        }
    }
    if (h_end != heads + 1) return;
    const T* kv = dkv + (size_t)t * dkv_stride;
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) {
        const float v = to_float(kv[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)rank + eps);
    if (page <= 0 || page >= num_pages) {
        if (tid == 0) atomicExch(&status[STATUS_BAD_PAGE], 1 + t);
        return;
    }
    CacheLayout L{1, page_size, D};
    T* kdst = cache + L.offset(page, 0, 0, p % page_size);
    T* vdst = cache + L.offset(page, 1, 0, p % page_size);
    if (pairs) {
        for (int i = tid * 2; i < D; i += blockDim.x * 2) {
            float a = 0.f, b = 0.f;
            if (i < rank) {
                load2(kv + i, a, b);
                a = a * inv * norm_w[i];
                b = b * inv * norm_w[i + 1];
            } else if (i < rank + rdim) {
                const int j = i - rank;
                load2(kv + i, a, b);
                if (j < rot) {
                        const float a0 = a, b0 = b;
                        rotate_pair(a0, b0, cs[j >> 1], sn[j >> 1], a, b);
                    }
            }
            store2(kdst + i, a, b);
            store2(vdst + i, a, b);
        }
        return;
    }
    for (int i = tid; i < D; i += blockDim.x) {
        float v = 0.f;
        if (i < rank) {
            v = to_float(kv[i]) * inv * norm_w[i];
        } else if (i < rank + rdim) {
            const int j = i - rank;
            v = to_float(kv[i]);
            if (j < rot) {
                const float other = to_float(kv[rank + (j ^ 1)]);
                float lo, hi;
                if (j & 1) { rotate_pair(other, v, cs[j >> 1], sn[j >> 1], lo, hi); v = hi; }
                else { rotate_pair(v, other, cs[j >> 1], sn[j >> 1], lo, hi); v = lo; }
            }
        }
        const T o = from_float<T>(v);
        kdst[i] = o;
        vdst[i] = o;
    }
}

extern "C" int latent_rows(const void* q_rot, long long qs_t, long long qs_h, const void* q_abs, const void* dkv,
                           long long dkv_stride, const float* norm_w, float eps, const int* positions, const int* token_entry,
                           const int* meta, int group, const float* inv_freq, int rot, void* q_out, void* cache, int dtype,
                           int T, int heads, int rank, int rdim, int D, int page_size, int num_pages, int store, int* status,
                           cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot % 2 || rot > rdim || rank + rdim > D || (rot && !inv_freq)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)rot * sizeof(float);
    const int elem = dtype == DT_F32 ? 4 : 2;
    const int pairs = rank % 2 == 0 && rdim % 2 == 0 && D % 2 == 0 && qs_t % 2 == 0 && qs_h % 2 == 0 && dkv_stride % 2 == 0 &&
                      (((uintptr_t)q_rot | (uintptr_t)q_abs | (uintptr_t)dkv | (uintptr_t)q_out | (uintptr_t)cache) % (2 * elem)) == 0;
    const int hpb = T >= 512 ? heads + 1 : 1, threads = hpb > 1 ? 256 : 128;
    const dim3 grid(T, (heads + 1 + hpb - 1) / hpb);
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, latent_rows_kernel<float>, grid, threads, smem, stream, (const float*)q_rot, qs_t,
                                      qs_h, (const float*)q_abs, (const float*)dkv, dkv_stride, norm_w, eps, positions, token_entry,
                                      meta, group, inv_freq, rot, (float*)q_out, (float*)cache, heads, rank, rdim, D, page_size,
                                      num_pages, store, pairs, hpb, status);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, latent_rows_kernel<__nv_bfloat16>, grid, threads, smem, stream,
                                  (const __nv_bfloat16*)q_rot, qs_t, qs_h, (const __nv_bfloat16*)q_abs, (const __nv_bfloat16*)dkv,
                                  dkv_stride, norm_w, eps, positions, token_entry, meta, group, inv_freq, rot,
                                  (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, heads, rank, rdim, D, page_size, num_pages, store,
                                  pairs, hpb, status);
}
