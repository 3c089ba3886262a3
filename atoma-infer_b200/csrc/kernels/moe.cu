// Kernels of routed experts: the router (float32 logits, softmax, the top choices and their weights), the (token,
// choice) pairs sorted by expert on the device, the experts' linears as grouped products over that order, and the
// weighted sum.  Storage is float32 or bfloat16, arithmetic float32; every output element is one accumulator running
// over k in order, so a token's result does not depend on what else is in the batch.
#include "common.cuh"

// ----------------------------------------------------------------------------- router
// One block per token: logits z_e = w_router[e] . h (float32, a warp per expert, lanes over k, summed in the fixed
// order of warp_sum); scores softmax(z); the `top` largest scores, ties to the lower index; weights = those scores
// divided by their sum (+ 1e-20).
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w, int* __restrict__ ids, float* __restrict__ wts,
                 const int* __restrict__ meta, int H, int E, int top, const float* __restrict__ bias, int over_chosen) {
    extern __shared__ float z[];  // E logits, then E scores that selection consumes
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const T* x = h + (size_t)t * H;
    const bool vec = H % 4 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
    for (int e = warp; e < E; e += nwarps) {
        const float* we = w + (size_t)e * H;
        float acc = 0.f;
        if (vec) {  // four columns a lane and step; the order of a logit's sum depends on H alone
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            for (int k = lane * 4; k < H; k += 128) {
                float xv[4], wv[4];
                load4(x + k, xv);
                load4(we + k, wv);
#pragma unroll
                for (int i = 0; i < 4; ++i) part[i] = fmaf(xv[i], wv[i], part[i]);
            }
            acc = (part[0] + part[1]) + (part[2] + part[3]);
        } else {
            for (int k = lane; k < H; k += 32) acc = fmaf(to_float(x[k]), we[k], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc + (bias ? bias[e] : 0.f);
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    float* s = z + E;
    if (over_chosen) {
        // the largest logits choose (ties to the lower index); the weights are the softmax over the chosen logits alone
        float first = 0.f, sum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (z[e] > bv) { bv = z[e]; best = e; }
            if (k == 0) first = bv;
            const float w_k = expf(bv - first);
            ids[(size_t)t * top + k] = best;
            wts[(size_t)t * top + k] = w_k;
            sum += w_k;
            z[best] = -INFINITY;
        }
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] = wts[(size_t)t * top + k] / sum;
        return;
    }
    float mx = -INFINITY, sum = 0.f;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, z[e]);
    for (int e = 0; e < E; ++e) { s[e] = expf(z[e] - mx); sum += s[e]; }
    for (int e = 0; e < E; ++e) s[e] = s[e] / sum;
    float chosen = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = 0;
        float bv = -1.f;
        for (int e = 0; e < E; ++e)
            if (s[e] > bv) { bv = s[e]; best = e; }
        ids[(size_t)t * top + k] = best;
        wts[(size_t)t * top + k] = bv;
        chosen += bv;
        s[best] = -2.f;
    }
    for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] = wts[(size_t)t * top + k] / (chosen + 1e-20f);
}

extern "C" int moe_route_biased(const void* h, int dtype, const float* w, const float* bias, int over_chosen, int* ids, float* wts,
                                const int* meta, int T, int H, int E, int top, cudaStream_t stream);

extern "C" int moe_route(const void* h, int dtype, const float* w, int* ids, float* wts, const int* meta, int T, int H, int E,
                         int top, cudaStream_t stream) {
    return moe_route_biased(h, dtype, w, nullptr, 0, ids, wts, meta, T, H, E, top, stream);
}

// bias (float32 [E], or null) is added to the logits.  over_chosen: the weights are the softmax over the chosen experts'
// logits alone (else: the softmax over all experts, the chosen scores divided by their sum).
extern "C" int moe_route_biased(const void* h, int dtype, const float* w, const float* bias, int over_chosen, int* ids, float* wts,
                                const int* meta, int T, int H, int E, int top, cudaStream_t stream) {
    if (T <= 0) return 0;
    const size_t smem = (size_t)2 * E * sizeof(float);
    if (smem > 48 * 1024 || top > E) return (int)cudaErrorInvalidValue;
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_route_kernel<float>, T, 256, smem, stream, (const float*)h, w, ids, wts,
                                      meta, H, E, top, bias, over_chosen);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_route_kernel<__nv_bfloat16>, T, 256, smem, stream,
                                  (const __nv_bfloat16*)h, w, ids, wts, meta, H, E, top, bias, over_chosen);
}

// ----------------------------------------------------------------------------- pairs sorted by expert
// One block.  offsets[e] .. offsets[e + 1] is expert e's stretch of `order`, which lists its pairs (token * top + choice)
// in ascending order.  A warp takes the experts e = warp, warp + warps, ...: it walks all pairs 32 at a time and
// places the matching ones by a ballot, once to count and once to write.
// `place` (optional): place[pair] = where the pair stands in `order`.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ place,
                const int* __restrict__ meta, int top, int E) {
    extern __shared__ int counts[];  // E + 1
    pdl_launch_dependents();
    pdl_wait();
    const int n = meta[META_NUM_TOKENS] * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        int c = 0;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            c += __popc(__ballot_sync(0xffffffffu, i < n && ids[i] == e));
        }
        if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { const int c = counts[e]; counts[e] = at; offsets[e] = at; at += c; }
        counts[E] = at;
        offsets[E] = at;
    }
    __syncthreads();
    for (int e = warp; e < E; e += nwarps) {
        int at = counts[e];
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < n && ids[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int to = at + __popc(m & ((1u << lane) - 1u));
                order[to] = i;
                if (place) place[i] = to;
            }
            at += __popc(m);
        }
    }
}

extern "C" int moe_sort(const int* ids, int* offsets, int* order, int* place, const int* meta, int top, int E,
                        cudaStream_t stream) {
    const size_t smem = (size_t)(E + 1) * sizeof(int);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return (int)launch_kernel(moe_sort_kernel, 1, 1024, smem, stream, ids, offsets, order, place, meta, top, E);
}

// ----------------------------------------------------------------------------- grouped products
// Row i of the sorted order belongs to expert e (offsets[e] <= i < offsets[e + 1]) and to pair order[i].
// mode 0: a[i, f] = silu(w[e, f] . x[pair / top]) * (w[e, F + f] . x[pair / top]) for f < F; w is [E, 2F, K], a is [pairs, F]
//         in sorted order.
// mode 1: y[pair, n] = w[e, n] . a[i]; w is [E, N, K], y is float32 [pairs, N] in pair order.
// A block takes GL_TM rows of ONE expert x GL_TN outputs; block x walks the experts' row tiles (at most
// ceil(pairs / GL_TM) + E of them), block y the output tiles.  x and w tiles go through shared memory GL_KC columns at
// a time; thread (ty, tx) owns rows ty * 2 .. and outputs tx * 4 ..
#define GL_TM 16
#define GL_TN 64
#define GL_KC 32
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
moe_grouped_linear_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ a_out, float* __restrict__ y_out,
                          const int* __restrict__ offsets, const int* __restrict__ order, int top, int E, int K, int N) {
    __shared__ float xs[GL_TM][GL_KC + 1];
    __shared__ float ws[(MODE == 0 ? 2 : 1) * GL_TN][GL_KC + 1];
    __shared__ int s_rows[GL_TM];
    __shared__ int s_e, s_first, s_count;
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x;
    if (tid == 0) {
        int tile = blockIdx.x, e = 0;
        s_e = -1;
        for (; e < E; ++e) {
            const int cnt = offsets[e + 1] - offsets[e], tiles = (cnt + GL_TM - 1) / GL_TM;
            if (tile < tiles) { s_e = e; s_first = offsets[e] + tile * GL_TM; s_count = min(GL_TM, cnt - tile * GL_TM); break; }
            tile -= tiles;
        }
    }
    __syncthreads();
    if (s_e < 0) return;
    const int e = s_e, first = s_first, rows = s_count, n0 = blockIdx.y * GL_TN;
    if (tid < GL_TM) s_rows[tid] = tid < rows ? (MODE == 0 ? order[first + tid] / top : first + tid) : -1;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 8
    const T* we = w + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    float acc[2][4], acc2[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = acc2[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += GL_KC) {
        const int kc = min(GL_KC, K - k0);
        __syncthreads();
        for (int idx = tid; idx < GL_TM * GL_KC; idx += 128) {
            const int m = idx / GL_KC, kk = idx % GL_KC, src = s_rows[m];
            xs[m][kk] = (src >= 0 && kk < kc) ? to_float(x[(size_t)src * K + k0 + kk]) : 0.f;
        }
        for (int idx = tid; idx < GL_TN * GL_KC; idx += 128) {
            const int j = idx / GL_KC, kk = idx % GL_KC;
            const bool ok = n0 + j < N && kk < kc;
            ws[j][kk] = ok ? to_float(we[(size_t)(n0 + j) * K + k0 + kk]) : 0.f;
            if (MODE == 0) ws[GL_TN + j][kk] = ok ? to_float(we[(size_t)(N + n0 + j) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
        for (int kk = 0; kk < kc; ++kk) {
            const float x0 = xs[ty * 2][kk], x1 = xs[ty * 2 + 1][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float wv = ws[tx * 4 + j][kk];
                acc[0][j] = fmaf(x0, wv, acc[0][j]);
                acc[1][j] = fmaf(x1, wv, acc[1][j]);
                if (MODE == 0) {
                    const float uv = ws[GL_TN + tx * 4 + j][kk];
                    acc2[0][j] = fmaf(x0, uv, acc2[0][j]);
                    acc2[1][j] = fmaf(x1, uv, acc2[1][j]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = ty * 2 + i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (MODE == 0) {
                const float g = acc[i][j];
                a_out[(size_t)(first + m) * N + n] = from_float<T>(g / (1.f + expf(-g)) * acc2[i][j]);
            } else {
                y_out[(size_t)order[first + m] * N + n] = acc[i][j];
            }
        }
    }
}

// x [tokens, H]; w_gate_up [E, 2F, H]; act [pairs, F] (sorted order); w_down [E, H, F]; y float32 [pairs, H] (pair order).
extern "C" int moe_grouped_ff(const void* x, const void* w_gate_up, void* act, const void* w_down, float* y, const int* offsets,
                              const int* order, int dtype, int T, int top, int E, int H, int F, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int tiles = (T * top + GL_TM - 1) / GL_TM + E;
    int err;
    if (dtype == DT_F32) {
        err = (int)launch_kernel(moe_grouped_linear_kernel<float, 0>, dim3(tiles, (F + GL_TN - 1) / GL_TN), 128, 0, stream,
                                 (const float*)x, (const float*)w_gate_up, (float*)act, (float*)nullptr, offsets, order, top, E, H, F);
        if (err) return err;
        return (int)launch_kernel(moe_grouped_linear_kernel<float, 1>, dim3(tiles, (H + GL_TN - 1) / GL_TN), 128, 0, stream,
                                  (const float*)act, (const float*)w_down, (float*)nullptr, y, offsets, order, top, E, F, H);
    }
    err = (int)launch_kernel(moe_grouped_linear_kernel<__nv_bfloat16, 0>, dim3(tiles, (F + GL_TN - 1) / GL_TN), 128, 0, stream,
                             (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate_up, (__nv_bfloat16*)act, (float*)nullptr, offsets,
                             order, top, E, H, F);
    if (err) return err;
    return (int)launch_kernel(moe_grouped_linear_kernel<__nv_bfloat16, 1>, dim3(tiles, (H + GL_TN - 1) / GL_TN), 128, 0, stream,
                              (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, (__nv_bfloat16*)nullptr, y, offsets, order,
                              top, E, F, H);
}

// ----------------------------------------------------------------------------- weighted sum
// out[t] = sum_k wts[t, k] * y[row of pair t * top + k] (+ shared[t]), choices in order, float32; a pair's row is the
// pair itself, or place[pair] when the rows are in sorted order.
template <typename TY, typename T>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place, const float* __restrict__ wts,
                   const T* __restrict__ shared, T* __restrict__ out, const int* __restrict__ meta, int top, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    if (t >= meta[META_NUM_TOKENS]) return;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const size_t row = place ? (size_t)place[(size_t)t * top + k] : (size_t)t * top + k;
            acc = fmaf(wts[(size_t)t * top + k], to_float(y[row * H + i]), acc);
        }
        if (shared) acc += to_float(shared[(size_t)t * H + i]);
        out[(size_t)t * H + i] = from_float<T>(acc);
    }
}

// y_dtype: float32 rows in pair order (place null), or rows of the compute type in sorted order with `place`.
extern "C" int moe_combine(const void* y, int y_dtype, const int* place, const float* wts, const void* shared, void* out,
                           int dtype, const int* meta, int T, int top, int H, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_combine_kernel<float, float>, T, threads, 0, stream, (const float*)y,
                                      place, wts, (const float*)shared, (float*)out, meta, top, H);
    if (y_dtype == DT_F32)
        return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_combine_kernel<float, __nv_bfloat16>, T, threads, 0, stream,
                                      (const float*)y, place, wts, (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, meta, top, H);
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_combine_kernel<__nv_bfloat16, __nv_bfloat16>, T, threads, 0, stream,
                                  (const __nv_bfloat16*)y, place, wts, (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, meta, top, H);
}

// ----------------------------------------------------------------------------- few pairs: a pair at a time
// Decode steps bring a handful of (token, choice) pairs, most of them alone with their expert: every pair streams its
// expert's rows itself.  A block takes one pair and PW_ROWS output rows; a warp takes a row at a time, its lanes 8
// columns (16 bytes) a step, several steps in flight; x waits in shared memory.  bfloat16 storage.
// gate/up: a[pair, f] = silu(w[e, f] . x[token]) * (w[e, F + f] . x[token]);  down: y[pair, n] = w[e, n] . a[pair] (float32).
#define PW_WARPS 8
#define PW_ROWS 32
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b, float acc) {
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
        acc = fmaf(fa.x, fb.x, acc);
        acc = fmaf(fa.y, fb.y, acc);
    }
    return acc;
}

template <int MODE>
__global__ void __launch_bounds__(PW_WARPS * 32)
moe_pair_linear_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ a_out,
                       float* __restrict__ y_out, const int* __restrict__ ids, const int* __restrict__ meta, int top, int K,
                       int N) {
    extern __shared__ __align__(16) unsigned char xs_raw[];
    uint4* xs = reinterpret_cast<uint4*>(xs_raw);  // K / 8 chunks
    const int pair = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool live = pair < meta[META_NUM_TOKENS] * top;  // (the step's metadata: written by no kernel of the step)
    pdl_launch_dependents();
    pdl_wait();
    if (!live) return;
    const int e = ids[pair];  // (the router's choice: a kernel of this step wrote it, so it is read after the wait)
    const int chunks = K / 8;
    const uint4* xrow = reinterpret_cast<const uint4*>(x + (size_t)(MODE == 0 ? pair / top : pair) * K);
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) xs[i] = xrow[i];
    __syncthreads();
    const __nv_bfloat16* we = w + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
    for (int r = warp; r < PW_ROWS; r += PW_WARPS) {
        const int n = blockIdx.x * PW_ROWS + r;
        if (n >= N) break;
        const uint4* g = reinterpret_cast<const uint4*>(we + (size_t)n * K);
        const uint4* u = reinterpret_cast<const uint4*>(we + (size_t)(N + n) * K);
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
        for (int c0 = lane; c0 < chunks; c0 += 128) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + j * 32;
                if (c < chunks) {
                    acc[j] = dot8(g[c], xs[c], acc[j]);
                    if (MODE == 0) acc2[j] = dot8(u[c], xs[c], acc2[j]);
                }
            }
        }
        float s = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (MODE == 0) {
            const float s2 = warp_sum((acc2[0] + acc2[1]) + (acc2[2] + acc2[3]));
            if (lane == 0) a_out[(size_t)pair * N + n] = __float2bfloat16_rn(s / (1.f + expf(-s)) * s2);
        } else if (lane == 0) {
            y_out[(size_t)pair * N + n] = s;
        }
    }
}

// x [tokens, H]; act [pairs, F] and y float32 [pairs, H], both in pair order.  H and F multiples of 8.
extern "C" int moe_pair_ff(const void* x, const void* w_gate_up, void* act, const void* w_down, float* y, const int* ids,
                           const int* meta, int T, int top, int H, int F, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H % 8 || F % 8 || (size_t)(H > F ? H : F) * 2 > 96 * 1024) return (int)cudaErrorInvalidValue;
    static size_t configured[2] = {0, 0};
    const size_t smem0 = (size_t)H * 2, smem1 = (size_t)F * 2;
    if (smem0 > 48 * 1024 && smem0 > configured[0]) {
        cudaError_t err = cudaFuncSetAttribute(moe_pair_linear_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem0);
        if (err != cudaSuccess) return (int)err;
        configured[0] = smem0;
    }
    if (smem1 > 48 * 1024 && smem1 > configured[1]) {
        cudaError_t err = cudaFuncSetAttribute(moe_pair_linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
        if (err != cudaSuccess) return (int)err;
        configured[1] = smem1;
    }
    int err = (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_pair_linear_kernel<0>, dim3((F + PW_ROWS - 1) / PW_ROWS, T * top),
                                     PW_WARPS * 32, smem0, stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate_up,
                                     (__nv_bfloat16*)act, (float*)nullptr, ids, meta, top, H, F);
    if (err) return err;
    return (int)launch_kernel_pdl((g_use_pdl & 5) != 0, moe_pair_linear_kernel<1>, dim3((H + PW_ROWS - 1) / PW_ROWS, T * top),
                                  PW_WARPS * 32, smem1, stream, (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down,
                                  (__nv_bfloat16*)nullptr, y, ids, meta, top, F, H);
}

// ----------------------------------------------------------------------------- many pairs: rows gathered for a library's grouped product
// xs[i] = x[order[i] / top] for the pairs in sorted order (16 bytes a thread; H * element size a multiple of 16).
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ xs, const int* __restrict__ order,
                       const int* __restrict__ meta, int top, int chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    if (i >= meta[META_NUM_TOKENS] * top) return;
    const uint4* src = x + (size_t)(order[i] / top) * chunks;
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) xs[(size_t)i * chunks + c] = src[c];
}

extern "C" int moe_gather_rows(const void* x, void* xs, const int* order, const int* meta, int T, int top, int row_bytes,
                               cudaStream_t stream) {
    if (T <= 0) return 0;
    if (row_bytes % 16) return (int)cudaErrorInvalidValue;
    return (int)launch_kernel(moe_gather_rows_kernel, T * top, 256, 0, stream, (const uint4*)x, (uint4*)xs, order, meta, top,
                              row_bytes / 16);
}
