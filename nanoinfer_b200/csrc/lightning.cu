// Lightning attention: linear attention with a fixed decay per head and a matrix state per request.
//
//   q = silu(W_q h), k = silu(W_k h)  [H, D];   v = silu(W_v h)  [H, V]          (the projections come in `proj`)
//   S_t = decay_h * S_(t-1) + k_t v_t^T  (S [D, V] per head, FP32, zero at a sequence's start);   o_t = S_t^T q_t
//   y = (o over all heads / sqrt(mean(o^2) + eps) * weight) * sigmoid(W_g h)
//
// Everything after the projections is FP32 whatever the tensors' type.
//
// lightning_chunk_kernel runs a request's tokens of this step in chunks of LT_C tokens.  With n tokens in a chunk,
// S0 the state before it and p[i] = decay^i (a table built by repeated multiplication, as the recurrence itself
// would):
//
//   A[t, j] = (q_t . k_j) p[t - j]                      for j <= t            (scores; no softmax)
//   o_t     = sum_(j <= t) A[t, j] v_j  +  p[t + 1] S0^T q_t
//   S       = p[n] S0 + sum_j p[n - 1 - j] k_j v_j^T
//
// which is the recurrence written out; only the order of the additions differs.  A single token is a chunk of
// one.  One block owns (request, head, LT_VT value columns): its tile of S stays in shared memory from the first
// chunk to the last and is read and written once per step.  All three products are register-tiled FP32 FMA
// loops over shared memory (the design keeps the scores and the state in 32 bits, so no tensor cores).
#include "common.cuh"

#define LT_C 64          // tokens per chunk
#define LT_VT 16         // value columns per block
#define LT_THREADS 256

__device__ __forceinline__ float lt_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
lightning_chunk_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state, long long state_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ slots, const float* __restrict__ decay,
                       float* __restrict__ out, int H, int D, int V) {
    extern __shared__ __align__(16) float sm[];
    const int DP = (D + 3) & ~3;             // rows padded to whole float4s (zeros)
    const int QS = DP + 4;                   // row stride of Qs / Ks: neighbouring rows start 4 banks apart
    float* Ss = sm;                          // [DP][LT_VT]
    float* Qs = Ss + DP * LT_VT;             // [LT_C][QS]
    float* Ks = Qs + LT_C * QS;              // [LT_C][QS]
    float* Vs = Ks + LT_C * QS;              // [LT_C][LT_VT]
    float* As = Vs + LT_C * LT_VT;           // [LT_C][LT_C + 4]
    float* pw = As + LT_C * (LT_C + 4);      // [LT_C + 1]
    constexpr int AS = LT_C + 4;

    const int tid = threadIdx.x;
    const int v0 = blockIdx.x * LT_VT, head = blockIdx.y, seq = blockIdx.z;
    const int vt = min(LT_VT, V - v0);
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t1 <= t0) return;
    float* S = state + (size_t)slots[seq] * state_stride + (size_t)head * D * V + v0;
    const float dec = decay[head];
    if (tid == 0) {
        float p = 1.0f;
        for (int i = 0; i <= LT_C; ++i) { pw[i] = p; p *= dec; }
    }
    for (int i = tid; i < DP * LT_VT; i += LT_THREADS) {
        const int d = i / LT_VT, v = i % LT_VT;
        Ss[i] = (d < D && v < vt) ? S[(size_t)d * V + v] : 0.f;
    }
    // the triangular tile of the score phase that this thread owns (4 x 4 scores; tiles on or below the diagonal)
    int a_ti = -1, a_ji = 0;
    if (tid < (LT_C / 4) * (LT_C / 4 + 1) / 2) {
        int ti = 0, rest = tid;
        while (rest > ti) { rest -= ti + 1; ++ti; }
        a_ti = ti;
        a_ji = rest;
    }
    const T* xq = proj + (size_t)head * D;
    const T* xk = proj + (size_t)(H + head) * D;
    const T* xv = proj + (size_t)2 * H * D + (size_t)head * V + v0;

    for (int c0 = t0; c0 < t1; c0 += LT_C) {
        const int n = min(LT_C, t1 - c0), n4 = (n + 3) & ~3;
        __syncthreads();                     // the chunk before is done with Qs, Ks, Vs, As (and pw, Ss are written)
        for (int i = tid; i < n4 * DP; i += LT_THREADS) {
            const int t = i / DP, d = i - t * DP;
            const bool in = t < n && d < D;
            const size_t at = (size_t)(c0 + t) * ld + d;
            Qs[t * QS + d] = in ? lt_silu(ni_to_float(xq[at])) : 0.f;
            Ks[t * QS + d] = in ? lt_silu(ni_to_float(xk[at])) : 0.f;
        }
        for (int i = tid; i < n4 * LT_VT; i += LT_THREADS) {
            const int t = i / LT_VT, v = i % LT_VT;
            Vs[i] = (t < n && v < vt) ? lt_silu(ni_to_float(xv[(size_t)(c0 + t) * ld + v])) : 0.f;
        }
        __syncthreads();
        // ---- scores: A[t, j] = (q_t . k_j) p[t - j], zero above the diagonal
        if (a_ti >= 0 && a_ti * 4 < n4) {
            float acc[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
            const float* qp = Qs + a_ti * 4 * QS;
            const float* kp = Ks + a_ji * 4 * QS;
            for (int d = 0; d < DP; d += 4) {
                float4 qv[4], kv[4];
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    qv[a] = *reinterpret_cast<const float4*>(qp + a * QS + d);
                    kv[a] = *reinterpret_cast<const float4*>(kp + a * QS + d);
                }
#pragma unroll
                for (int a = 0; a < 4; ++a)
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        acc[a][b] = fmaf(qv[a].x, kv[b].x, acc[a][b]);
                        acc[a][b] = fmaf(qv[a].y, kv[b].y, acc[a][b]);
                        acc[a][b] = fmaf(qv[a].z, kv[b].z, acc[a][b]);
                        acc[a][b] = fmaf(qv[a].w, kv[b].w, acc[a][b]);
                    }
            }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int t = a_ti * 4 + a, j = a_ji * 4 + b;
                    As[t * AS + j] = j <= t ? acc[a][b] * pw[t - j] : 0.f;
                }
        }
        __syncthreads();
        // ---- read-out: o_t = sum_(j <= t) A[t, j] v_j + p[t + 1] S0^T q_t; thread = 4 tokens x 1 value column
        {
            const int v = tid % LT_VT, tg = tid / LT_VT;         // 16 groups of 4 tokens
            if (tg * 4 < n4) {
                float intra[4] = {0.f, 0.f, 0.f, 0.f}, inter[4] = {0.f, 0.f, 0.f, 0.f};
                const int j_end = tg * 4 + 4;                     // scores beyond the diagonal are zero
                for (int j = 0; j < j_end; j += 4) {
                    float4 av[4];
#pragma unroll
                    for (int a = 0; a < 4; ++a) av[a] = *reinterpret_cast<const float4*>(As + (tg * 4 + a) * AS + j);
                    const float w0 = Vs[j * LT_VT + v], w1 = Vs[(j + 1) * LT_VT + v], w2 = Vs[(j + 2) * LT_VT + v],
                                w3 = Vs[(j + 3) * LT_VT + v];
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        intra[a] = fmaf(av[a].x, w0, intra[a]);
                        intra[a] = fmaf(av[a].y, w1, intra[a]);
                        intra[a] = fmaf(av[a].z, w2, intra[a]);
                        intra[a] = fmaf(av[a].w, w3, intra[a]);
                    }
                }
                for (int d = 0; d < DP; d += 4) {
                    float4 qv[4];
#pragma unroll
                    for (int a = 0; a < 4; ++a) qv[a] = *reinterpret_cast<const float4*>(Qs + (tg * 4 + a) * QS + d);
                    const float s0 = Ss[d * LT_VT + v], s1 = Ss[(d + 1) * LT_VT + v], s2 = Ss[(d + 2) * LT_VT + v],
                                s3 = Ss[(d + 3) * LT_VT + v];
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        inter[a] = fmaf(qv[a].x, s0, inter[a]);
                        inter[a] = fmaf(qv[a].y, s1, inter[a]);
                        inter[a] = fmaf(qv[a].z, s2, inter[a]);
                        inter[a] = fmaf(qv[a].w, s3, inter[a]);
                    }
                }
                if (v < vt) {
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        const int t = tg * 4 + a;
                        if (t < n) out[(size_t)(c0 + t) * H * V + (size_t)head * V + v0 + v] = fmaf(pw[t + 1], inter[a], intra[a]);
                    }
                }
            }
        }
        __syncthreads();
        // ---- the values take their decay to the chunk's end: v_j <- p[n - 1 - j] v_j
        for (int i = tid; i < n * LT_VT; i += LT_THREADS) Vs[i] *= pw[n - 1 - i / LT_VT];
        __syncthreads();
        // ---- state: S = p[n] S0 + sum_j k_j (p[n - 1 - j] v_j)^T; thread = 1 value column x every 16th row group of 4
        {
            const int v = tid % LT_VT;
            const float pn = pw[n];
            for (int d = (tid / LT_VT) * 4; d < DP; d += (LT_THREADS / LT_VT) * 4) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int j = 0; j < n; ++j) {
                    const float4 kv = *reinterpret_cast<const float4*>(Ks + j * QS + d);
                    const float w = Vs[j * LT_VT + v];
                    acc[0] = fmaf(kv.x, w, acc[0]);
                    acc[1] = fmaf(kv.y, w, acc[1]);
                    acc[2] = fmaf(kv.z, w, acc[2]);
                    acc[3] = fmaf(kv.w, w, acc[3]);
                }
#pragma unroll
                for (int a = 0; a < 4; ++a) Ss[(d + a) * LT_VT + v] = fmaf(pn, Ss[(d + a) * LT_VT + v], acc[a]);
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < D * LT_VT; i += LT_THREADS) {
        const int d = i / LT_VT, v = i % LT_VT;
        if (v < vt) S[(size_t)d * V + v] = Ss[i];
    }
}

// y[t, :] = o[t, :] / sqrt(mean(o[t]^2) + eps) * weight * sigmoid(gate[t, :]); o FP32 [T, N], the gate's columns lie
// in proj at col0, y in the activations' type.  One block per token.
template <typename T>
__global__ void lightning_gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, int ld, int col0,
                                            const float* __restrict__ weight, float eps, T* __restrict__ y, int N) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float* row = o + (size_t)t * N;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss += row[i] * row[i];
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)N + eps);
    const T* g = proj + (size_t)t * ld + col0;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float gate = 1.0f / (1.0f + expf(-ni_to_float(g[i])));
        y[(size_t)t * N + i] = ni_from_float<T>(row[i] * inv * weight[i] * gate);
    }
}

static size_t lt_smem_bytes(int D) {
    const int DP = (D + 3) & ~3;
    return ((size_t)DP * LT_VT + 2 * (size_t)LT_C * (DP + 4) + (size_t)LT_C * LT_VT + (size_t)LT_C * (LT_C + 4) + LT_C + 1) *
           sizeof(float);
}

// proj [T, ld] with columns q (H D) | k (H D) | v (H V) | ...; state FP32 [slots, state_stride] holding S [H, D, V] of
// every request; decay FP32 [H]; out FP32 [T, H V].  The state advances by the step's tokens.
NI_EXPORT int ni_lightning_recurrence(const void* proj, int dtype, int ld, float* state, long long state_stride,
                                      const int* cu_q, const int* slots, const float* decay, float* out, int n_tokens,
                                      int n_seqs, int H, int D, int V, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return NI_OK;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + H * V || state_stride < (long long)H * D * V) return NI_ERR_BAD_ARGUMENT;
    const size_t smem = lt_smem_bytes(D);
    if (smem > 200 * 1024 || H > 65535 || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((V + LT_VT - 1) / LT_VT, H, n_seqs);
#define LAUNCH(T)                                                                                                        \
    do {                                                                                                                 \
        cudaFuncSetAttribute(lightning_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        lightning_chunk_kernel<T><<<grid, LT_THREADS, smem, stream>>>((const T*)proj, ld, state, state_stride, cu_q,    \
                                                                      slots, decay, out, H, D, V);                       \
    } while (0)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_lightning_gated_norm(const float* o, const void* proj, int dtype, int ld, int col0, const float* weight,
                                      float eps, void* y, int n_tokens, int N, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (N <= 0 || col0 < 0 || col0 + N > ld) return NI_ERR_BAD_ARGUMENT;
    const int threads = N >= 1024 ? 256 : 128;
#define LAUNCH(T) \
    lightning_gated_norm_kernel<T><<<n_tokens, threads, 0, stream>>>(o, (const T*)proj, ld, col0, weight, eps, (T*)y, N)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
