// Recurrent mixers whose state is a matrix per head or per channel and whose decay differs from row to row:
//  * gated linear attention: per head S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, a_t = sigmoid(z_t)^(1/tau);
//  * the selective scan of the Mamba kind: per channel c and state n, S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c u_c B_n,
//    y_c = sum_n S[c, n] C_n + D_c u_c, times silu(z_c);
//  * the norm per head with a weight shared by the heads, times silu(gate), behind the first.
// Storage of projections is float32 or bfloat16; states, decays, step sizes, gates and norms are float32 always.  A
// request's tokens run in order from its state slot (pass 0), or, for long portions, cut into chunks of time that run
// side by side: pass 1 runs every chunk but the last from a zero state and leaves its end state and what its decays
// amount to, a small kernel chains the chunks' start states in order, pass 3 runs every chunk again from its start
// state and writes the outputs, the last chunk the slot.  Every sum runs in an order that depends on the sizes only.
#include "common.cuh"

#define REC_TT 16  // tokens staged in shared memory at a time

int g_use_pdl = 1;
extern "C" void kernels_set_pdl(int mode) { g_use_pdl = mode; }

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

// Two float32 operations in one instruction (sm_100): the recurrences' arithmetic is bound by instruction issue, and a
// pair of neighbouring rows comes out of one 16-byte load of shared memory as two such operands.  Each half is the plain
// IEEE operation, rounded to nearest.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)),
          "l"(reinterpret_cast<const unsigned long long&>(c)));
    return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 d;
    asm("mul.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<unsigned long long&>(d))
        : "l"(reinterpret_cast<const unsigned long long&>(a)), "l"(reinterpret_cast<const unsigned long long&>(b)));
    return d;
}

// ----------------------------------------------------------------------------- gated linear attention
// q, k [T, heads * N], v [T, heads * P]: slices of wider rows (strides in elements); z float32 [T, heads * N], the decay's
// logits before their bias.  state [slots][heads][N][P]; o float32 [T, heads * P].
// One block per (head x column block, entry[, chunk]).  Thread (pl, r) keeps NPT rows n = r * NPT .. of CPT neighbouring
// columns in registers (a row's k, a and q are loaded once for all of them); R threads (a power of two, neighbouring
// lanes) share the columns; rows beyond N see k = q = 0 and stay zero.  P is a multiple of CPT.  An output is the sum of
// the even rows' products plus the sum of the odd rows', each in ascending order, then the R threads' sums by halving.
template <typename T>
struct alignas(4 * sizeof(T)) Raw4 { T x[4]; };  // four stored values, loaded at once

template <typename T, int NPT, bool WRITE_O, int CPT>
__global__ void __launch_bounds__(256, NPT <= 16 ? 2 : 1)
gla_scan_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k, long long k_stride,
                const T* __restrict__ v, long long v_stride, const float* __restrict__ z, long long z_stride,
                const float* __restrict__ z_bias, float inv_tau, float q_scale, float* __restrict__ state,
                long long slot_stride, float* __restrict__ o, const int* __restrict__ meta,
                const int* __restrict__ cu_tokens, const int* __restrict__ slots, int heads, int P, int N, int R, int PB,
                int col_blocks, int pass, int chunk_len, int max_chunks, float* __restrict__ scratch,
                float* __restrict__ decay, int vec, int mode) {
    extern __shared__ __align__(16) float sm[];
    // mode bit 0: no logits; every row of head h decays by the constant z_bias[h].  bit 1: q, k and v pass through SiLU.
    const bool fixed = mode & 1, act = mode & 2;
    const int SL = R > 1 ? NPT + 4 : NPT, NL = R * NPT, NP = R * SL;  // row n lies at (n / NPT) * SL + n % NPT
    float* qs = sm;                     // [REC_TT][NP]
    float* ks = qs + REC_TT * NP;       // [REC_TT][NP]
    float* as = ks + REC_TT * NP;       // [REC_TT][NP]
    float* vs = as + REC_TT * NP;       // [REC_TT][PB]
    const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks, e = blockIdx.y, c = blockIdx.z;
    pdl_launch_dependents();
    pdl_wait();
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int first = cu_tokens[e], count = cu_tokens[e + 1] - first;
    const int nchunks = pass == 0 ? 1 : (count + chunk_len - 1) / chunk_len;
    if (c >= nchunks || (pass == 1 && c == nchunks - 1)) return;
    const int t0 = first + (pass == 0 ? 0 : c * chunk_len), t1 = pass == 0 ? first + count : min(first + count, t0 + chunk_len);
    const int tid = threadIdx.x, pl = tid / R, r = tid % R, p = cb * PB + pl * CPT;
    const bool real = pl * CPT < PB && p < P;  // all CPT columns, or none
    const size_t HS = (size_t)N * P;
    float* slot_state = state + (size_t)slots[e] * slot_stride + (size_t)h * HS;
    float* chunk_state = scratch ? scratch + (((size_t)e * max_chunks + c) * heads + h) * HS : nullptr;
    float2 S[CPT][NPT / 2], prod[WRITE_O ? 1 : NPT / 2];
    const float* init = pass == 0 ? slot_state : (pass == 3 ? chunk_state : nullptr);
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = r * NPT + i;
        float row[CPT];
#pragma unroll
        for (int j = 0; j < CPT; ++j) row[j] = 0.f;
        if (init && real && n < N) {
            const float* src = init + (size_t)n * P + p;
            if constexpr (CPT == 4) { const float4 x = *reinterpret_cast<const float4*>(src); row[0] = x.x, row[1] = x.y, row[2] = x.z, row[3] = x.w; }
            else if constexpr (CPT == 2) { const float2 x = *reinterpret_cast<const float2*>(src); row[0] = x.x, row[1] = x.y; }
            else row[0] = src[0];
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j) (i & 1 ? S[j][i / 2].y : S[j][i / 2].x) = row[j];
        if constexpr (!WRITE_O) prod[i / 2] = make_float2(1.f, 1.f);
    }
    for (int tb = t0; tb < t1; tb += REC_TT) {
        const int nt = min(REC_TT, t1 - tb);
        __syncthreads();  // the previous tile is no longer read
        if (CPT > 1 && vec) {  // (the one-column kernels, which run steps of few tokens, stay small: more blocks at a time)
            // four neighbouring rows (or columns) an item, two items a thread at a time, every load ahead of the first use
            const int QI = NL / 4, qitems = nt * QI, VI = PB / 4, vitems = nt * VI;
            for (int i0 = tid; i0 < qitems; i0 += 2 * blockDim.x) {
                Raw4<T> rq[2], rk[2];
                float4 rz[2];
                int at[2], hn4[2];
                bool in[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int idx = i0 + u * blockDim.x, tt = idx / QI, n = (idx % QI) * 4;
                    at[u] = idx < qitems ? tt * NP + (n / NPT) * SL + n % NPT : -1;
                    in[u] = idx < qitems && n < N;
                    hn4[u] = h * N + n;
                    if (in[u]) {
                        const size_t t = (size_t)(tb + tt), hn = (size_t)h * N + n;
                        rq[u] = *reinterpret_cast<const Raw4<T>*>(q + t * q_stride + hn);
                        rk[u] = *reinterpret_cast<const Raw4<T>*>(k + t * k_stride + hn);
                        if (!fixed) rz[u] = *reinterpret_cast<const float4*>(z + t * z_stride + hn);
                    }
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (at[u] < 0) continue;
                    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f), k4 = q4, a4 = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (in[u]) {
                        // (the bias is the same for every token: it stays in the first-level cache)
                        float qv[4], kv[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            qv[j] = to_float(rq[u].x[j]), kv[j] = to_float(rk[u].x[j]);
                            if (act) qv[j] = silu_f(qv[j]), kv[j] = silu_f(kv[j]);
                        }
                        q4 = make_float4(qv[0] * q_scale, qv[1] * q_scale, qv[2] * q_scale, qv[3] * q_scale);
                        k4 = make_float4(kv[0], kv[1], kv[2], kv[3]);
                        if (fixed) {
                            const float a = z_bias[h];
                            a4 = make_float4(a, a, a, a);
                        } else {
                        const float4 rb = z_bias ? *reinterpret_cast<const float4*>(z_bias + hn4[u]) : make_float4(0.f, 0.f, 0.f, 0.f);
                        a4 = make_float4(expf(-softplus_f(-(rz[u].x + rb.x)) * inv_tau), expf(-softplus_f(-(rz[u].y + rb.y)) * inv_tau),
                                         expf(-softplus_f(-(rz[u].z + rb.z)) * inv_tau), expf(-softplus_f(-(rz[u].w + rb.w)) * inv_tau));
                        }
                    }
                    *reinterpret_cast<float4*>(qs + at[u]) = q4;
                    *reinterpret_cast<float4*>(ks + at[u]) = k4;
                    *reinterpret_cast<float4*>(as + at[u]) = a4;
                }
            }
            for (int i0 = tid; i0 < vitems; i0 += 2 * blockDim.x) {
                Raw4<T> rv[2];
                int at[2];
                bool in[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int idx = i0 + u * blockDim.x, tt = idx / VI, pc = cb * PB + (idx % VI) * 4;
                    at[u] = idx < vitems ? idx * 4 : -1;
                    in[u] = idx < vitems && pc < P;
                    if (in[u]) rv[u] = *reinterpret_cast<const Raw4<T>*>(v + (size_t)(tb + tt) * v_stride + (size_t)h * P + pc);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (at[u] < 0) continue;
                    float vv4[4] = {0.f, 0.f, 0.f, 0.f};
                    if (in[u]) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) vv4[j] = act ? silu_f(to_float(rv[u].x[j])) : to_float(rv[u].x[j]);
                    }
                    *reinterpret_cast<float4*>(vs + at[u]) = make_float4(vv4[0], vv4[1], vv4[2], vv4[3]);
                }
            }
        } else {
        for (int idx = tid; idx < nt * NL; idx += blockDim.x) {
            const int tt = idx / NL, n = idx % NL, at = tt * NP + (n / NPT) * SL + n % NPT;
            const size_t t = (size_t)(tb + tt);
            float qv = 0.f, kv = 0.f, av = 1.f;
            if (n < N) {
                qv = to_float(q[t * q_stride + (size_t)h * N + n]);
                kv = to_float(k[t * k_stride + (size_t)h * N + n]);
                if (act) qv = silu_f(qv), kv = silu_f(kv);
                qv *= q_scale;
                if (fixed) {
                    av = z_bias[h];
                } else {
                    // sigmoid(x)^(1/tau) = exp(-softplus(-x) / tau)
                    const float x = z[t * z_stride + (size_t)h * N + n] + (z_bias ? z_bias[(size_t)h * N + n] : 0.f);
                    av = expf(-softplus_f(-x) * inv_tau);
                }
            }
            qs[at] = qv;
            ks[at] = kv;
            as[at] = av;
        }
        for (int idx = tid; idx < nt * PB; idx += blockDim.x) {
            const int tt = idx / PB, pc = cb * PB + idx % PB;
            const float x = pc < P ? to_float(v[(size_t)(tb + tt) * v_stride + (size_t)h * P + pc]) : 0.f;
            vs[idx] = act ? silu_f(x) : x;
        }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float2 vv[CPT], acc[CPT];
            {
                const float* vt = vs + tt * PB + (pl * CPT < PB ? pl * CPT : 0);
                float x[CPT];
                if constexpr (CPT == 4) { const float4 y = *reinterpret_cast<const float4*>(vt); x[0] = y.x, x[1] = y.y, x[2] = y.z, x[3] = y.w; }
                else if constexpr (CPT == 2) { const float2 y = *reinterpret_cast<const float2*>(vt); x[0] = y.x, x[1] = y.y; }
                else x[0] = vt[0];
#pragma unroll
                for (int j = 0; j < CPT; ++j) vv[j] = make_float2(x[j], x[j]), acc[j] = make_float2(0.f, 0.f);
            }
            const float* kt = ks + tt * NP + r * SL;
            const float* at = as + tt * NP + r * SL;
            const float* qt = qs + tt * NP + r * SL;
#pragma unroll
            for (int i = 0; i < NPT; i += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kt + i);
                const float4 a4 = *reinterpret_cast<const float4*>(at + i);
                const float2 k01 = make_float2(k4.x, k4.y), k23 = make_float2(k4.z, k4.w);
                const float2 a01 = make_float2(a4.x, a4.y), a23 = make_float2(a4.z, a4.w);
                float2 q01 = make_float2(0.f, 0.f), q23 = q01;
                if constexpr (WRITE_O) {
                    const float4 q4 = *reinterpret_cast<const float4*>(qt + i);
                    q01 = make_float2(q4.x, q4.y), q23 = make_float2(q4.z, q4.w);
                } else {
                    prod[i / 2] = mul2(prod[i / 2], a01);
                    prod[i / 2 + 1] = mul2(prod[i / 2 + 1], a23);
                }
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    S[j][i / 2] = fma2(a01, S[j][i / 2], mul2(k01, vv[j]));
                    S[j][i / 2 + 1] = fma2(a23, S[j][i / 2 + 1], mul2(k23, vv[j]));
                    if constexpr (WRITE_O) {
                        acc[j] = fma2(S[j][i / 2], q01, acc[j]);
                        acc[j] = fma2(S[j][i / 2 + 1], q23, acc[j]);
                    }
                }
            }
            if constexpr (WRITE_O) {
                float sum[CPT];
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    sum[j] = acc[j].x + acc[j].y;
                    for (int s = R >> 1; s > 0; s >>= 1) sum[j] += __shfl_xor_sync(0xffffffffu, sum[j], s);
                }
                if (real && r == 0) {
                    float* dst = o + (size_t)(tb + tt) * heads * P + (size_t)h * P + p;
                    if constexpr (CPT == 4) *reinterpret_cast<float4*>(dst) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                    else if constexpr (CPT == 2) *reinterpret_cast<float2*>(dst) = make_float2(sum[0], sum[1]);
                    else dst[0] = sum[0];
                }
            }
        }
    }
    float* fin = pass == 1 ? chunk_state + (size_t)heads * HS /* the next chunk's place */
                           : ((pass == 0 || c == nchunks - 1) ? slot_state : nullptr);
    if (fin && real) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = r * NPT + i;
            if (n < N) {
                float row[CPT];
#pragma unroll
                for (int j = 0; j < CPT; ++j) row[j] = i & 1 ? S[j][i / 2].y : S[j][i / 2].x;
                float* dst = fin + (size_t)n * P + p;
                if constexpr (CPT == 4) *reinterpret_cast<float4*>(dst) = make_float4(row[0], row[1], row[2], row[3]);
                else if constexpr (CPT == 2) *reinterpret_cast<float2*>(dst) = make_float2(row[0], row[1]);
                else dst[0] = row[0];
            }
        }
    }
    if constexpr (!WRITE_O) if (pass == 1 && cb == 0 && pl == 0) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = r * NPT + i;
            if (n < N) decay[(((size_t)e * max_chunks + c) * heads + h) * N + n] = i & 1 ? prod[i / 2].y : prod[i / 2].x;
        }
    }
}

// scratch[e, 0] = the slot's state; scratch[e, c] = decay[e, c - 1] (a factor per row) * scratch[e, c - 1] + scratch[e, c].
__global__ void __launch_bounds__(256)
gla_chunk_states_kernel(const float* __restrict__ state, long long slot_stride, float* __restrict__ scratch,
                        const float* __restrict__ decay, const int* __restrict__ meta, const int* __restrict__ cu_tokens,
                        const int* __restrict__ slots, int heads, int N, int P, int chunk_len, int max_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, e = blockIdx.y;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int count = cu_tokens[e + 1] - cu_tokens[e], nchunks = (count + chunk_len - 1) / chunk_len;
    const long long HS = (long long)N * P;
    const float* src = state + (size_t)slots[e] * slot_stride + (size_t)h * HS;
    for (long long i = (long long)blockIdx.z * blockDim.x + threadIdx.x; i < HS; i += (long long)gridDim.z * blockDim.x) {
        const int n = (int)(i / P);
        float s = src[i];
        scratch[(((size_t)e * max_chunks) * heads + h) * HS + i] = s;
        for (int c = 1; c < nchunks; ++c) {
            float* at = scratch + (((size_t)e * max_chunks + c) * heads + h) * HS + i;
            s = fmaf(decay[(((size_t)e * max_chunks + c - 1) * heads + h) * N + n], s, *at);
            *at = s;
        }
    }
}

// Rows a thread keeps and threads a column (or channel): the least padding, then 16 or 32 rows a thread.  Columns a
// block: those of up to 256 threads, ``cpt`` neighbouring columns each.
static bool rec_geometry(int N, int P, int* NPT_out, int* R_out, int* PB_out, int cpt = 1) {
    static const int sizes[] = {16, 32, 8, 64};  // in order of preference among equal paddings
    long best = -1;
    for (int k = 0; k < 4; ++k) {
        const int npt = sizes[k];
        int R = 1;
        while (R * npt < N) R *= 2;
        if (R > 32) continue;
        const long cost = (long)R * npt;
        if (best < 0 || cost < best) best = cost, *NPT_out = npt, *R_out = R;
    }
    if (best < 0) return false;
    int pb = 256 / *R_out * cpt;  // up to 256 threads a block
    if (pb > P) pb = P;
    *PB_out = pb;
    return true;
}

extern "C" size_t gla_scan_scratch_floats(int S, int heads, int N, int P, int max_chunks) {
    return (size_t)S * max_chunks * heads * ((size_t)N * P + N);
}

extern "C" int gla_scan_mode(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                             int dtype, const float* z, long long z_stride, const float* z_bias, float tau, float q_scale,
                             float* state, long long slot_stride, float* o, const int* meta, const int* cu_tokens, const int* slots,
                             int S, int heads, int N, int P, int chunk_len, int max_chunks, float* scratch, int mode,
                             cudaStream_t stream);

extern "C" int gla_scan(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                        int dtype, const float* z, long long z_stride, const float* z_bias, float tau, float q_scale,
                        float* state, long long slot_stride, float* o, const int* meta, const int* cu_tokens, const int* slots,
                        int S, int heads, int N, int P, int chunk_len, int max_chunks, float* scratch, cudaStream_t stream) {
    return gla_scan_mode(q, q_stride, k, k_stride, v, v_stride, dtype, z, z_stride, z_bias, tau, q_scale, state, slot_stride, o, meta,
                         cu_tokens, slots, S, heads, N, P, chunk_len, max_chunks, scratch, 0, stream);
}

// mode bit 0: the decay is a constant per head, z_bias[h] (float32 [heads]; z is not read); bit 1: q, k and v pass through
// SiLU as they are loaded.
extern "C" int gla_scan_mode(const void* q, long long q_stride, const void* k, long long k_stride, const void* v, long long v_stride,
                             int dtype, const float* z, long long z_stride, const float* z_bias, float tau, float q_scale,
                             float* state, long long slot_stride, float* o, const int* meta, const int* cu_tokens, const int* slots,
                             int S, int heads, int N, int P, int chunk_len, int max_chunks, float* scratch, int mode,
                             cudaStream_t stream) {
    if (S <= 0) return 0;
    if ((mode & 1) ? !z_bias : !z) return (int)cudaErrorInvalidValue;
    int NPT = 0, R = 0, PB = 0;
    if (tau <= 0.f || !rec_geometry(N, P, &NPT, &R, &PB)) return (int)cudaErrorInvalidValue;
    const bool chunked = chunk_len > 0 && max_chunks > 1 && scratch;
    // Columns a thread: with chunks of time there are blocks enough, and a row's k, a and q serve four (or two) columns;
    // a step of few tokens per entry keeps one, for as many blocks as can be.  Vector accesses want their alignment.
    auto aligned = [&](int n) {
        return P % n == 0 && slot_stride % n == 0 && ((uintptr_t)state | (uintptr_t)o | (uintptr_t)scratch) % (4 * n) == 0;
    };
    const int CPT = !chunked ? 1 : (NPT <= 16 && aligned(4) ? 4 : (NPT <= 32 && aligned(2) ? 2 : 1));
    rec_geometry(N, P, &NPT, &R, &PB, CPT);
    // tiles of q, k, decay logits and v in items of four: rows and columns in fours, every row's slice on its vector's boundary
    const uintptr_t esz = dtype == DT_F32 ? 4 : 2;
    const int vec = N % 4 == 0 && P % 4 == 0 && PB % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 &&
                    z_stride % 4 == 0 && ((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) % (4 * esz) == 0 &&
                    ((mode & 1) || ((uintptr_t)z | (uintptr_t)z_bias) % 16 == 0);
    const int col_blocks = (P + PB - 1) / PB, threads = ((PB / CPT * R + 31) / 32) * 32;
    const size_t smem = (size_t)(3 * REC_TT * R * (R > 1 ? NPT + 4 : NPT) + REC_TT * PB) * sizeof(float);
    if (smem > 96 * 1024) return (int)cudaErrorInvalidValue;
    float* decay = scratch ? scratch + (size_t)S * max_chunks * heads * (size_t)N * P : nullptr;
    const float inv_tau = 1.f / tau;
#define GLA_LAUNCH(TT, K, W, C, pass, chunks)                                                                               \
    {                                                                                                                      \
        static size_t configured = 0;                                                                                      \
        if (smem > 48 * 1024 && smem > configured) {                                                                       \
            cudaError_t ce = cudaFuncSetAttribute(gla_scan_kernel<TT, K, W, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (ce != cudaSuccess) return (int)ce;                                                                         \
            configured = smem;                                                                                             \
        }                                                                                                                  \
        err = (int)launch_kernel(gla_scan_kernel<TT, K, W, C>, dim3(heads * col_blocks, S, chunks), threads, smem, stream, (const TT*)q, q_stride, \
                                 (const TT*)k, k_stride, (const TT*)v, v_stride, z, z_stride, z_bias, inv_tau, q_scale, state, \
                                 slot_stride, o, meta, cu_tokens, slots, heads, P, N, R, PB, col_blocks, pass, chunk_len,     \
                                 max_chunks, scratch, decay, vec, mode);                                                   \
    }
#define GLA_CASE(TT, K, W, pass, chunks)                                                                                    \
    case K:                                                                                                                \
        if (CPT == 4) { if constexpr (K <= 16) GLA_LAUNCH(TT, K, W, 4, pass, chunks) }                                     \
        else if (CPT == 2) { if constexpr (K <= 32) GLA_LAUNCH(TT, K, W, 2, pass, chunks) }                                \
        else GLA_LAUNCH(TT, K, W, 1, pass, chunks)                                                                         \
        break;
#define GLA_PASS(TT, W, pass, chunks)                                                                                       \
    switch (NPT) { GLA_CASE(TT, 8, W, pass, chunks) GLA_CASE(TT, 16, W, pass, chunks) GLA_CASE(TT, 32, W, pass, chunks) GLA_CASE(TT, 64, W, pass, chunks) }
    int err = 0;
    if (!chunked) {
        if (dtype == DT_F32) { GLA_PASS(float, true, 0, 1) } else { GLA_PASS(__nv_bfloat16, true, 0, 1) }
        return err;
    }
    if (dtype == DT_F32) { GLA_PASS(float, false, 1, max_chunks) } else { GLA_PASS(__nv_bfloat16, false, 1, max_chunks) }
    if (err) return err;
    const int zblocks = (int)(((long long)N * P + 1023) / 1024);
    err = (int)launch_kernel(gla_chunk_states_kernel, dim3(heads, S, zblocks), 256, 0, stream, (const float*)state, slot_stride,
                             scratch, (const float*)decay, meta, cu_tokens, slots, heads, N, P, chunk_len, max_chunks);
    if (err) return err;
    if (dtype == DT_F32) { GLA_PASS(float, true, 3, max_chunks) } else { GLA_PASS(__nv_bfloat16, true, 3, max_chunks) }
    return err;
#undef GLA_PASS
#undef GLA_LAUNCH
#undef GLA_CASE
}

// ----------------------------------------------------------------------------- norm per head, shared weight, gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w * silu(g[t, h, :]); o float32 [T, heads * P], g a slice of
// wider rows, w float32 [P].  A warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, long long g_stride, const float* __restrict__ w,
                      float eps, T* __restrict__ out, const int* __restrict__ meta, int heads, int P) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, lane = threadIdx.x & 31, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= meta[META_NUM_TOKENS] || h >= heads) return;
    const float* row = o + ((size_t)t * heads + h) * P;
    const T* gate = g + (size_t)t * g_stride + (size_t)h * P;
    float ss = 0.f;
    for (int i = lane; i < P; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)P + eps);
    T* dst = out + ((size_t)t * heads + h) * P;
    for (int i = lane; i < P; i += 32) dst[i] = from_float<T>(row[i] * inv * w[i] * silu_f(to_float(gate[i])));
}

extern "C" int head_norm_gate(const float* o, const void* g, int dtype, long long g_stride, const float* w, float eps, void* out,
                              const int* meta, int T, int heads, int P, cudaStream_t stream) {
    if (T <= 0) return 0;
    const dim3 grid(T, (heads + 3) / 4);
    if (dtype == DT_F32)
        return (int)launch_kernel(head_norm_gate_kernel<float>, grid, 128, 0, stream, o, (const float*)g, g_stride, w, eps,
                                  (float*)out, meta, heads, P);
    return (int)launch_kernel(head_norm_gate_kernel<__nv_bfloat16>, grid, 128, 0, stream, o, (const __nv_bfloat16*)g, g_stride, w,
                              eps, (__nv_bfloat16*)out, meta, heads, P);
}

// ----------------------------------------------------------------------------- selective scan
// u [T, inner] (after convolution and activation), zg [T, inner] (the gate's input): slices of wider rows; dt_raw float32
// [T, inner] (softplus(dt_raw + dt_bias) is taken here); B at bc, C at bc + N of a row of bc_stride elements; a_log [inner, N];
// state [slots][inner][N]; out [T, inner] = (sum_n S[c, n] C_n + D_c u_c) * silu(zg_c).
// One block per (channel block, entry[, chunk]).  Thread (c, r) keeps NPT states n = r * NPT .. of channel c, as pairs of
// neighbouring states that one two-wide instruction updates.  y is the even states' sum plus the odd states', each in
// ascending order, then the R threads' sums by halving.  B and C of 16 tokens are staged in shared memory; the channel's
// own u, step size and gate input of those tokens go straight into the thread's registers.
#define LOG2E_F 1.4426950408889634f

// 2^x for x <= 0 by the hardware's instruction alone (what exp2f runs for arguments in the normal range; a result below
// the smallest normal number is zero, which a decay of that size is for every state that float32 holds).
__device__ __forceinline__ float ex2_nonpositive(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T, int NPT, bool WRITE_Y>
__global__ void __launch_bounds__(256)
selective_scan_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ dt_raw,
                      const float* __restrict__ dt_bias, const T* __restrict__ bc, long long bc_stride,
                      const T* __restrict__ zg, long long z_stride, const float* __restrict__ a_log,
                      const float* __restrict__ d_skip, float* __restrict__ state, long long slot_stride, T* __restrict__ out,
                      const int* __restrict__ meta, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                      int inner, int N, int R, int CPB, int pass, int chunk_len, int max_chunks, float* __restrict__ scratch,
                      float* __restrict__ dt_sums) {
    extern __shared__ __align__(16) float sm[];
    const int SL = R > 1 ? NPT + 4 : NPT, NL = R * NPT, NP = R * SL;
    float* Bs = sm;                      // [REC_TT][NP]
    float* Cs = Bs + REC_TT * NP;        // [REC_TT][NP]
    const int e = blockIdx.y, ch = blockIdx.z;
    const int tid = threadIdx.x, cl = tid / R, r = tid % R, c = blockIdx.x * CPB + cl;
    const bool real = cl < CPB && c < inner;
    // the weights come before the wait: no kernel writes them
    float2 A2[NPT / 2];  // A log2(e), pairs of neighbouring states
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = r * NPT + i;
        const float a = (real && n < N) ? -expf(a_log[(size_t)c * N + n]) * LOG2E_F : 0.f;
        if (i & 1) A2[i / 2].y = a; else A2[i / 2].x = a;
    }
    const float dskip = real ? d_skip[c] : 0.f, dtb = real ? dt_bias[c] : 0.f;
    pdl_launch_dependents();
    pdl_wait();
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int first = cu_tokens[e], count = cu_tokens[e + 1] - first;
    const int nchunks = pass == 0 ? 1 : (count + chunk_len - 1) / chunk_len;
    if (ch >= nchunks || (pass == 1 && ch == nchunks - 1)) return;
    const int t0 = first + (pass == 0 ? 0 : ch * chunk_len), t1 = pass == 0 ? first + count : min(first + count, t0 + chunk_len);
    const size_t HS = (size_t)inner * N;
    float* slot_state = state + (size_t)slots[e] * slot_stride;
    float* chunk_state = scratch ? scratch + ((size_t)e * max_chunks + ch) * HS : nullptr;
    const float* init = pass == 0 ? slot_state : (pass == 3 ? chunk_state : nullptr);
    float2 S[NPT / 2];
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
        const int n = r * NPT + i;
        const float s0 = (init && real && n < N) ? init[(size_t)c * N + n] : 0.f;
        if (i & 1) S[i / 2].y = s0; else S[i / 2].x = s0;
    }
    float dt_sum = 0.f;
    for (int tb = t0; tb < t1; tb += REC_TT) {
        const int nt = min(REC_TT, t1 - tb);
        // this thread's channel of the tile's tokens, straight into registers: every load is on its way before the
        // first is used (the R threads of a channel read the same addresses)
        T ur[REC_TT], zr[REC_TT];
        float dr[REC_TT];
#pragma unroll
        for (int tt = 0; tt < REC_TT; ++tt) {
            const bool in = real && tt < nt;
            const size_t t = (size_t)(tb + tt);
            ur[tt] = in ? u[t * u_stride + c] : from_float<T>(0.f);
            dr[tt] = in ? dt_raw[t * inner + c] : 0.f;
            if (WRITE_Y) zr[tt] = in ? zg[t * z_stride + c] : from_float<T>(0.f);
        }
        __syncthreads();
        for (int idx = tid; idx < nt * NL; idx += blockDim.x) {
            const int tt = idx / NL, n = idx % NL, at = tt * NP + (n / NPT) * SL + n % NPT;
            const T* row = bc + (size_t)(tb + tt) * bc_stride;
            Bs[at] = n < N ? to_float(row[n]) : 0.f;
            Cs[at] = n < N ? to_float(row[N + n]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int tt = 0; tt < REC_TT; ++tt) {
            if (tt >= nt) break;
            const float uv = to_float(ur[tt]), step = real ? softplus_f(dr[tt] + dtb) : 0.f;
            const float dx = step * uv;
            const float* Bt = Bs + tt * NP + r * SL;
            const float* Ct = Cs + tt * NP + r * SL;
            const float2 st2 = make_float2(step, step), dx2 = make_float2(dx, dx);
            float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < NPT / 2; i += 2) {  // two pairs of neighbouring states a round
                const float4 b4 = *reinterpret_cast<const float4*>(Bt + 2 * i);
                float2 ea = mul2(st2, A2[i]), eb = mul2(st2, A2[i + 1]);
                ea = make_float2(ex2_nonpositive(ea.x), ex2_nonpositive(ea.y));
                eb = make_float2(ex2_nonpositive(eb.x), ex2_nonpositive(eb.y));
                S[i] = fma2(ea, S[i], mul2(dx2, make_float2(b4.x, b4.y)));
                S[i + 1] = fma2(eb, S[i + 1], mul2(dx2, make_float2(b4.z, b4.w)));
                if (WRITE_Y) {
                    const float4 c4 = *reinterpret_cast<const float4*>(Ct + 2 * i);
                    acc2 = fma2(S[i], make_float2(c4.x, c4.y), acc2);
                    acc2 = fma2(S[i + 1], make_float2(c4.z, c4.w), acc2);
                }
            }
            float acc = acc2.x + acc2.y;  // the even states' sum plus the odd states'
            if (WRITE_Y) {
                for (int s = R >> 1; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
                if (real && r == 0) {
                    const float y = fmaf(dskip, uv, acc);
                    out[(size_t)(tb + tt) * inner + c] = from_float<T>(y * silu_f(to_float(zr[tt])));
                }
            }
            dt_sum += step;
        }
    }
    float* fin = pass == 1 ? chunk_state + HS : ((pass == 0 || ch == nchunks - 1) ? slot_state : nullptr);
    if (fin && real) {
#pragma unroll
        for (int i = 0; i < NPT; ++i) {
            const int n = r * NPT + i;
            if (n < N) fin[(size_t)c * N + n] = (i & 1) ? S[i / 2].y : S[i / 2].x;
        }
    }
    if (pass == 1 && real && r == 0) dt_sums[((size_t)e * max_chunks + ch) * inner + c] = dt_sum;
}

// scratch[e, 0] = the slot's state; scratch[e, c] = exp(A * (sum of the steps of chunk c - 1)) * scratch[e, c - 1] + scratch[e, c].
__global__ void __launch_bounds__(256)
selective_chunk_states_kernel(const float* __restrict__ state, long long slot_stride, float* __restrict__ scratch,
                              const float* __restrict__ dt_sums, const float* __restrict__ a_log, const int* __restrict__ meta,
                              const int* __restrict__ cu_tokens, const int* __restrict__ slots, int inner, int N, int chunk_len,
                              int max_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const int e = blockIdx.y;
    if (e >= meta[META_NUM_ENTRIES]) return;
    const int count = cu_tokens[e + 1] - cu_tokens[e], nchunks = (count + chunk_len - 1) / chunk_len;
    const long long HS = (long long)inner * N, i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= HS) return;
    const int c = (int)(i / N);
    const float a2 = -expf(a_log[i]) * LOG2E_F;
    float s = state[(size_t)slots[e] * slot_stride + i];
    scratch[((size_t)e * max_chunks) * HS + i] = s;
    for (int k = 1; k < nchunks; ++k) {
        float* at = scratch + ((size_t)e * max_chunks + k) * HS + i;
        s = fmaf(exp2f(a2 * dt_sums[((size_t)e * max_chunks + k - 1) * inner + c]), s, *at);
        *at = s;
    }
}

extern "C" size_t selective_scan_scratch_floats(int S, int inner, int N, int max_chunks) {
    return (size_t)S * max_chunks * ((size_t)inner * N + inner);
}

extern "C" int selective_scan(const void* u, long long u_stride, const float* dt_raw, const float* dt_bias, const void* bc,
                              long long bc_stride, const void* zg, long long z_stride, int dtype, const float* a_log,
                              const float* d_skip, float* state, long long slot_stride, void* out, const int* meta,
                              const int* cu_tokens, const int* slots, int S, int inner, int N, int chunk_len, int max_chunks,
                              float* scratch, cudaStream_t stream) {
    if (S <= 0) return 0;
    int NPT = 0, R = 0, CPB = 0;
    if (!rec_geometry(N, inner, &NPT, &R, &CPB)) return (int)cudaErrorInvalidValue;
    if (CPB * R > 128) CPB = 128 / R > 0 ? 128 / R : 1;  // 128 threads a block: more blocks for few requests
    const int blocks = (inner + CPB - 1) / CPB, threads = ((CPB * R + 31) / 32) * 32;
    const size_t smem = (size_t)(2 * REC_TT * R * (R > 1 ? NPT + 4 : NPT)) * sizeof(float);
    if (smem > 96 * 1024) return (int)cudaErrorInvalidValue;
    float* dt_sums = scratch ? scratch + (size_t)S * max_chunks * (size_t)inner * N : nullptr;
#define SEL_CASE(TT, K, W, pass, chunks)                                                                                    \
    case K: {                                                                                                              \
        static size_t configured = 0;                                                                                      \
        if (smem > 48 * 1024 && smem > configured) {                                                                       \
            cudaError_t ce = cudaFuncSetAttribute(selective_scan_kernel<TT, K, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (ce != cudaSuccess) return (int)ce;                                                                         \
            configured = smem;                                                                                             \
        }                                                                                                                  \
        err = (int)launch_kernel(selective_scan_kernel<TT, K, W>, dim3(blocks, S, chunks), threads, smem, stream, (const TT*)u, u_stride, \
                                 dt_raw, dt_bias, (const TT*)bc, bc_stride, (const TT*)zg, z_stride, a_log, d_skip, state,       \
                                 slot_stride, (TT*)out, meta, cu_tokens, slots, inner, N, R, CPB, pass, chunk_len, max_chunks,   \
                                 scratch, dt_sums);                                                                        \
        break;                                                                                                             \
    }
#define SEL_PASS(TT, W, pass, chunks)                                                                                       \
    switch (NPT) { SEL_CASE(TT, 8, W, pass, chunks) SEL_CASE(TT, 16, W, pass, chunks) SEL_CASE(TT, 32, W, pass, chunks) SEL_CASE(TT, 64, W, pass, chunks) }
    int err = 0;
    if (chunk_len <= 0 || max_chunks <= 1 || !scratch) {
        if (dtype == DT_F32) { SEL_PASS(float, true, 0, 1) } else { SEL_PASS(__nv_bfloat16, true, 0, 1) }
        return err;
    }
    if (dtype == DT_F32) { SEL_PASS(float, false, 1, max_chunks) } else { SEL_PASS(__nv_bfloat16, false, 1, max_chunks) }
    if (err) return err;
    const long long HS = (long long)inner * N;
    err = (int)launch_kernel(selective_chunk_states_kernel, dim3((unsigned)((HS + 255) / 256), S), 256, 0, stream,
                             (const float*)state, slot_stride, scratch, (const float*)dt_sums, a_log, meta, cu_tokens, slots,
                             inner, N, chunk_len, max_chunks);
    if (err) return err;
    if (dtype == DT_F32) { SEL_PASS(float, true, 3, max_chunks) } else { SEL_PASS(__nv_bfloat16, true, 3, max_chunks) }
    return err;
#undef SEL_PASS
#undef SEL_CASE
}
