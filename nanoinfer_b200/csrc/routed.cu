// A routed feed-forward: every token chooses a few of many small gated units ("experts").
//
//   route     z = W_router x, s = softmax(z) over all experts - or s = sigmoid(z), each expert on its own -, all FP32;
//             the `top` experts with the largest s + bias are chosen (ties: the lower index), their weights are s
//             (optionally divided by their sum).  Experts numbered n_real and above are identity experts: their
//             output is x itself.
//   unit      an expert is W_down act(W_gate x, W_up x) with act(g, u) = g' * sigmoid(slope * g') * (u' + shift),
//             g' = min(r g, limit), u' = clamp(r u, -limit, limit): limit = infinity, slope = 1, shift = 0, r = 1 is
//             silu(g) * u; r is a number per row - the token's weight where a design multiplies the expert's INPUT by
//             it (both products are linear in the input, so the factor is applied to their results, in FP32)
//   layout    the (token, choice) pairs are laid out expert by expert (layout + scatter; where a pair lands
//             inside its expert's stretch is decided by an atomic counter and changes no result, since every
//             row is computed on its own)
//   few rows  bfloat16, fewer pairs than experts: one warp per (pair, output) streams the expert's row with 16-byte
//             loads (expert_rows: silu(gate) * up, or the plain product); no layout is needed
//             (with as many pairs as experts or more, the part multiplies with ALL experts' matrices in one
//             skinny product instead, which reads every matrix once, and the combination picks the chosen rows)
//   many rows one launch multiplies every stretch with its expert's matrix (expert_gemm: each output element is
//             ONE chain of fused multiply-adds over k ascending, in FP32, whatever the row's place in a tile)
//   combine   y[t] = sum over the token's choices, in the order they were chosen, of weight * (expert output
//             or x[t]), FP32
//
// Nothing is decided on the host: grids cover the most rows there can be, and the counts stay on the device.
#include "common.cuh"

#define RT_MAX_EXPERTS 256
#define RT_ROUTE_WARPS 8

// One block per token: the token's row is widened to FP32 in shared memory once, the warps share the experts'
// dot products (each one warp's sum in a fixed order), and the first warp does the softmax and the choice.
template <typename T>
__global__ void __launch_bounds__(RT_ROUTE_WARPS * 32)
route_kernel(const T* __restrict__ x, const float* __restrict__ w_router,
             const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights,
             int* __restrict__ counts, int n_tokens, int d, int n_all, int n_real, int top,
             int renormalize, int sigmoid_scores, float* __restrict__ all_scores) {
    extern __shared__ __align__(16) float xs[];          // [d]
    __shared__ float choice[RT_MAX_EXPERTS];
    __shared__ float score[RT_MAX_EXPERTS];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const T* xr = x + (size_t)t * d;
    for (int k = threadIdx.x; k < d; k += blockDim.x) xs[k] = ni_to_float(xr[k]);
    __syncthreads();
    for (int e = w; e < n_all; e += RT_ROUTE_WARPS) {
        const float* wr = w_router + (size_t)e * d;
        float acc = 0.f;
        if ((d & 3) == 0) {
            const float4* w4 = reinterpret_cast<const float4*>(wr);
            const float4* x4 = reinterpret_cast<const float4*>(xs);
            for (int k = lane; k < (d >> 2); k += 32) {
                const float4 a = x4[k], b = w4[k];
                acc = fmaf(a.x, b.x, acc);
                acc = fmaf(a.y, b.y, acc);
                acc = fmaf(a.z, b.z, acc);
                acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (int k = lane; k < d; k += 32) acc = fmaf(xs[k], wr[k], acc);
        }
        acc = ni_warp_sum(acc);
        if (lane == 0) score[e] = acc;
    }
    __syncthreads();
    if (w != 0) return;
    float inv = 1.0f;
    if (!sigmoid_scores) {
        float m = -INFINITY;
        for (int e = lane; e < n_all; e += 32) m = fmaxf(m, score[e]);
        m = ni_warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < n_all; e += 32) {
            const float p = expf(score[e] - m);
            score[e] = p;
            sum += p;
        }
        sum = ni_warp_sum(sum);
        inv = 1.0f / sum;
    }
    for (int e = lane; e < n_all; e += 32) {
        const float s = sigmoid_scores ? 1.0f / (1.0f + expf(-score[e])) : score[e] * inv;
        score[e] = s;
        choice[e] = s + (bias ? bias[e] : 0.f);
        if (all_scores && e < n_real) all_scores[(size_t)t * n_real + e] = s;      // every real expert's score, chosen or not
    }
    __syncwarp();
    float wsum = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < n_all; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; arg = e; }       // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= n_all) arg = j;                      // only if every remaining score is NaN: keep indices valid
        const float s = score[arg];
        wsum += s;
        if (lane == 0) {
            ids[(size_t)t * top + j] = arg;
            weights[(size_t)t * top + j] = s;
            choice[arg] = -INFINITY;
            if (arg < n_real && counts) atomicAdd(&counts[arg], 1);
        }
        __syncwarp();
    }
    if (renormalize && lane < top) weights[(size_t)t * top + lane] /= wsum;   // top <= 32 when this is asked
}

// offsets[e] = first row of expert e's stretch, tile_first[e] = first row tile (tiles of `tile_rows` rows);
// the counts and the cursors are left zero for the next use.
__global__ void layout_kernel(int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ tile_first,
                              int* __restrict__ cursor, int n_real, int tile_rows) {
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < n_real; ++e) {
            const int c = counts[e];
            offsets[e] = rows;
            tile_first[e] = tiles;
            rows += c;
            tiles += (c + tile_rows - 1) / tile_rows;
            counts[e] = 0;
            cursor[e] = 0;
        }
        offsets[n_real] = rows;
        tile_first[n_real] = tiles;
    }
}

__global__ void scatter_kernel(const int* __restrict__ ids, const int* __restrict__ offsets, int* __restrict__ cursor,
                               int* __restrict__ row_of_pair, int* __restrict__ token_of_row, int n_pairs, int top,
                               int n_real, const float* __restrict__ weights, float* __restrict__ weight_of_row) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    const int e = ids[p];
    if (e >= n_real) {
        row_of_pair[p] = -1;
        return;
    }
    const int row = offsets[e] + atomicAdd(&cursor[e], 1);
    row_of_pair[p] = row;
    token_of_row[row] = p / top;
    if (weight_of_row) weight_of_row[row] = weights[p];
}

// out[row, :] = a[row or its token, :] . w[expert of the row]^T for every row of every expert's stretch.
// 64 x 64 tiles, 16 x 16 threads with 4 x 4 outputs each; ACT: the matrix holds gate rows [0, N) and up rows
// [N, 2N) and the result is silu(gate) * up.
// limit, slope, shift of a unit's activation, and the row's factor (see the head of this file)
struct RtAct {
    float limit, slope, shift;
};
__device__ __forceinline__ float rt_act(float g, float u, const RtAct a, float r) {
    g = fminf(g * r, a.limit);
    u = fminf(fmaxf(u * r, -a.limit), a.limit);
    return g / (1.0f + expf(-a.slope * g)) * (u + a.shift);
}

#define RT_BM 64
#define RT_BN 64
#define RT_BK 16

template <typename T, bool ACT>
__global__ void __launch_bounds__(256)
expert_gemm_kernel(const T* __restrict__ a, const int* __restrict__ token_of_row, const T* __restrict__ w,
                   T* __restrict__ out, const int* __restrict__ offsets, const int* __restrict__ tile_first,
                   int n_real, int N, int K, RtAct act, const float* __restrict__ row_scale) {
    __shared__ float as[RT_BK][RT_BM + 4];
    __shared__ float ws[RT_BK][RT_BN + 4];
    __shared__ float us[ACT ? RT_BK : 1][RT_BN + 4];
    __shared__ int src_row[RT_BM];
    __shared__ int s_expert;
    const int tile = blockIdx.y;
    if (tile >= tile_first[n_real]) return;
    if (threadIdx.x == 0) {
        int e = 0;
        while (tile >= tile_first[e + 1]) ++e;
        s_expert = e;
    }
    __syncthreads();
    const int e = s_expert;
    const int row_lo = offsets[e] + (tile - tile_first[e]) * RT_BM, row_hi = offsets[e + 1];
    if (threadIdx.x < RT_BM) {
        const int r = row_lo + threadIdx.x;
        src_row[threadIdx.x] = r < row_hi ? (token_of_row ? token_of_row[r] : r) : -1;
    }
    __syncthreads();
    const T* we = w + (size_t)e * (ACT ? 2 : 1) * N * K;
    const int n0 = blockIdx.x * RT_BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4], acu[ACT ? 4 : 1][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.f;
            if (ACT) acu[i][j] = 0.f;
        }
    for (int k0 = 0; k0 < K; k0 += RT_BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = threadIdx.x + 256 * q;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            const int sr = src_row[r];
            as[kk][r] = (sr >= 0 && k < K) ? ni_to_float(a[(size_t)sr * K + k]) : 0.f;
            ws[kk][r] = (n0 + r < N && k < K) ? ni_to_float(we[(size_t)(n0 + r) * K + k]) : 0.f;
            if (ACT) us[kk][r] = (n0 + r < N && k < K) ? ni_to_float(we[(size_t)(N + n0 + r) * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < RT_BK; ++kk) {
            float av[4], bv[4], uv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = as[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j] = ws[kk][tx * 4 + j];
                if (ACT) uv[j] = us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
                    if (ACT) acu[i][j] = fmaf(av[i], uv[j], acu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = row_lo + ty * 4 + i;
        if (r >= row_hi) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (ACT) {
                // the products are rounded to the activations' type first, as a separate product would leave them
                const float g = ni_to_float(ni_from_float<T>(v)), u = ni_to_float(ni_from_float<T>(acu[i][j]));
                v = rt_act(g, u, act, row_scale ? row_scale[r] : 1.0f);
            }
            out[(size_t)r * N + n] = ni_from_float<T>(v);
        }
    }
}

// Few rows, bfloat16: one warp per (pair, output).  a: the tokens' rows [T, K] (GATHER: pair p reads row
// p / top) or the pairs' own rows [P, K]; K a multiple of 8.
template <bool ACT>
__global__ void expert_rows_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ out, const int* __restrict__ ids, int n_pairs, int top,
                                   int gather, int n_real, int N, int K, RtAct act, const float* __restrict__ row_scale) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int p = blockIdx.y;
    if (warp >= N) return;
    const int e = ids[p];
    if (e >= n_real) return;
    const __nv_bfloat16* ar = a + (size_t)(gather ? p / top : p) * K;
    const __nv_bfloat16* wg = w + ((size_t)e * (ACT ? 2 : 1) * N + warp) * K;
    const __nv_bfloat16* wu = wg + (size_t)N * K;
    float g = 0.f, u = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 av = *reinterpret_cast<const uint4*>(ar + k);
        const uint4 gv = *reinterpret_cast<const uint4*>(wg + k);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 af = __bfloat1622float2(a2[i]), gf = __bfloat1622float2(g2[i]);
            g = fmaf(af.x, gf.x, g);
            g = fmaf(af.y, gf.y, g);
        }
        if (ACT) {
            const uint4 uv = *reinterpret_cast<const uint4*>(wu + k);
            const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 af = __bfloat1622float2(a2[i]), uf = __bfloat1622float2(u2[i]);
                u = fmaf(af.x, uf.x, u);
                u = fmaf(af.y, uf.y, u);
            }
        }
    }
    g = ni_warp_sum(g);
    if (ACT) {
        u = ni_warp_sum(u);
        g = __bfloat162float(__float2bfloat16_rn(g));
        u = __bfloat162float(__float2bfloat16_rn(u));
        g = rt_act(g, u, act, row_scale ? row_scale[p] : 1.0f);
    }
    if (lane == 0) out[(size_t)p * N + warp] = __float2bfloat16_rn(g);
}

// y[t, :] = sum_j weights[t, j] * (expert rows: z[row of pair (t, j), :];  identity experts: x[t, :]), FP32
// all_experts > 0: z holds a row for every (token, expert), [T, all_experts, d], and pair p's row is t * all_experts + ids[p]
template <typename T>
__global__ void combine_kernel(const T* __restrict__ z, const T* __restrict__ x, const int* __restrict__ ids,
                               const float* __restrict__ weights, const int* __restrict__ row_of_pair,
                               float* __restrict__ y, int d, int top, int n_real, int all_experts, int unit_real,
                               int accumulate) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = accumulate ? y[(size_t)t * d + c] : 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = t * top + j;
            const int e = ids[p];
            const float wgt = (unit_real && e < n_real) ? 1.0f : weights[p];
            const int row = all_experts > 0 ? t * all_experts + e : (row_of_pair ? row_of_pair[p] : p);
            const float v = e >= n_real ? ni_to_float(x[(size_t)t * d + c]) : ni_to_float(z[(size_t)row * d + c]);
            acc = fmaf(wgt, v, acc);
        }
        y[(size_t)t * d + c] = acc;
    }
}

// The same sum, divided by its root mean square, times a gain, added into the FP32 stream: h[t] += y / rms(y) * gain
// (the norm that an arrangement puts on a sublayer's output, without a round trip of y through memory).
template <typename T>
__global__ void combine_add_normed_kernel(const T* __restrict__ z, const T* __restrict__ x, const int* __restrict__ ids,
                                          const float* __restrict__ weights, const int* __restrict__ row_of_pair,
                                          float* __restrict__ h, const float* __restrict__ gain, float eps, int d, int top,
                                          int n_real, int all_experts, int unit_real) {
    extern __shared__ float ys[];          // [d]
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < top; ++j) {
            const int p = t * top + j;
            const int e = ids[p];
            const int row = all_experts > 0 ? t * all_experts + e : (row_of_pair ? row_of_pair[p] : p);
            const float v = e >= n_real ? ni_to_float(x[(size_t)t * d + c]) : ni_to_float(z[(size_t)row * d + c]);
            acc = fmaf((unit_real && e < n_real) ? 1.0f : weights[p], v, acc);
        }
        ys[c] = acc;
        ss += acc * acc;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) h[(size_t)t * d + c] += ys[c] * inv * gain[c];
}

// The same, 16 bytes per thread (widths that are multiples of 8 bfloat16 or 4 float values; at most 256 choices):
// the token's weights and rows are looked up once into shared memory.
template <typename T>
__global__ void combine_add_normed_vec_kernel(const T* __restrict__ z, const T* __restrict__ x, const int* __restrict__ ids,
                                              const float* __restrict__ weights, const int* __restrict__ row_of_pair,
                                              float* __restrict__ h, const float* __restrict__ gain, float eps, int d, int top,
                                              int n_real, int all_experts, int unit_real) {
    constexpr int V = NiVec16<T>::N;
    extern __shared__ __align__(16) float ys[];          // [d]
    __shared__ float scratch[32];
    __shared__ float s_w[RT_MAX_EXPERTS];
    __shared__ int s_row[RT_MAX_EXPERTS];
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < top; j += blockDim.x) {
        const int p = t * top + j, e = ids[p];
        s_w[j] = (unit_real && e < n_real) ? 1.0f : weights[p];
        s_row[j] = e >= n_real ? -1 : (all_experts > 0 ? t * all_experts + e : (row_of_pair ? row_of_pair[p] : p));
    }
    __syncthreads();
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < d; c += blockDim.x * V) {
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.f;
        for (int j = 0; j < top; ++j) {
            const int row = s_row[j];
            float v[V];
            NiVec16<T>::load((row < 0 ? x + (size_t)t * d : z + (size_t)row * d) + c, v);
            const float wgt = s_w[j];
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = fmaf(wgt, v[k], acc[k]);
        }
#pragma unroll
        for (int k = 0; k < V; ++k) {
            ys[c + k] = acc[k];
            ss += acc[k] * acc[k];
        }
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        float a[4], g[4];
        NiVec16<float>::load(h + (size_t)t * d + c, a);
        NiVec16<float>::load(gain + c, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] += ys[c + k] * inv * g[k];
        NiVec16<float>::store(h + (size_t)t * d + c, a);
    }
}

NI_EXPORT int ni_route(const void* x, int dtype, const float* w_router, const float* bias, int* ids, float* weights,
                       int* counts, int n_tokens, int d, int n_all, int n_real, int top, int renormalize,
                       int sigmoid_scores, float* all_scores, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || n_all <= 0 || n_real < 0 || n_real > n_all || top <= 0 || top > n_all) return NI_ERR_BAD_ARGUMENT;
    if (n_all > RT_MAX_EXPERTS || (renormalize && top > 32)) return NI_ERR_UNSUPPORTED_SIZE;
    if (d > 12000) return NI_ERR_UNSUPPORTED_SIZE;                    // the row lies in shared memory as FP32
    const size_t smem = (size_t)d * sizeof(float);
    if (dtype == NI_DTYPE_F32)
        route_kernel<float><<<n_tokens, RT_ROUTE_WARPS * 32, smem, stream>>>((const float*)x, w_router, bias, ids, weights,
                                                                           counts, n_tokens, d, n_all, n_real, top, renormalize,
                                                                           sigmoid_scores, all_scores);
    else if (dtype == NI_DTYPE_BF16)
        route_kernel<__nv_bfloat16><<<n_tokens, RT_ROUTE_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)x, w_router, bias,
                                                                                   ids, weights, counts, n_tokens, d, n_all,
                                                                                   n_real, top, renormalize, sigmoid_scores,
                                                                                   all_scores);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// counts [n_real] (zero before the route kernel ran, zero again afterwards), offsets and tile_first [n_real + 1],
// cursor [n_real], row_of_pair [n_pairs], token_of_row [n_pairs]
NI_EXPORT int ni_route_layout(const int* ids, int* counts, int* offsets, int* tile_first, int* cursor, int* row_of_pair,
                              int* token_of_row, int n_pairs, int top, int n_real, const float* weights,
                              float* weight_of_row, cudaStream_t stream) {
    if (n_pairs <= 0) return NI_OK;
    if (n_real < 0 || top <= 0) return NI_ERR_BAD_ARGUMENT;
    layout_kernel<<<1, 32, 0, stream>>>(counts, offsets, tile_first, cursor, n_real, RT_BM);
    scatter_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(ids, offsets, cursor, row_of_pair, token_of_row, n_pairs, top,
                                                              n_real, weights, weight_of_row);
    NI_RETURN_LAUNCH_STATUS();
}

// act != 0: w is [n_real, 2 N, K] (gate rows, then up rows) and out = silu(gate) * up
NI_EXPORT int ni_expert_gemm(const void* a, int dtype, const int* token_of_row, const void* w, void* out,
                             const int* offsets, const int* tile_first, int n_pairs, int n_real, int N, int K, int act,
                             float limit, float slope, float shift, const float* row_scale, cudaStream_t stream) {
    if (n_pairs <= 0 || n_real <= 0 || N <= 0) return NI_OK;
    if (K <= 0) return NI_ERR_BAD_ARGUMENT;
    const int max_tiles = (n_pairs + RT_BM - 1) / RT_BM + (n_real < n_pairs ? n_real : n_pairs);
    dim3 grid((N + RT_BN - 1) / RT_BN, max_tiles);
    if (grid.y > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    const RtAct ra = {limit, slope, shift};
#define LAUNCH(T, ACT)                                                                                             \
    expert_gemm_kernel<T, ACT><<<grid, 256, 0, stream>>>((const T*)a, token_of_row, (const T*)w, (T*)out, offsets, \
                                                         tile_first, n_real, N, K, ra, row_scale)
    if (dtype == NI_DTYPE_F32) { if (act) LAUNCH(float, true); else LAUNCH(float, false); }
    else if (dtype == NI_DTYPE_BF16) { if (act) LAUNCH(__nv_bfloat16, true); else LAUNCH(__nv_bfloat16, false); }
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_expert_rows(const void* a, const void* w, void* out, const int* ids, int n_pairs, int top, int gather,
                             int n_real, int N, int K, int act, float limit, float slope, float shift,
                             const float* row_scale, cudaStream_t stream) {
    if (n_pairs <= 0 || n_real <= 0 || N <= 0) return NI_OK;
    if (K <= 0 || top <= 0) return NI_ERR_BAD_ARGUMENT;
    if (K % 8 || n_pairs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((N + 7) / 8, n_pairs);
    const RtAct ra = {limit, slope, shift};
    if (act)
        expert_rows_kernel<true><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                           (__nv_bfloat16*)out, ids, n_pairs, top, gather, n_real, N, K, ra, row_scale);
    else
        expert_rows_kernel<false><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)w,
                                                            (__nv_bfloat16*)out, ids, n_pairs, top, gather, n_real, N, K, ra, row_scale);
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_route_combine_add_normed(const void* z, const void* x, int dtype, const int* ids, const float* weights,
                                          const int* row_of_pair, float* h, const float* gain, float eps, int n_tokens,
                                          int d, int top, int n_real, int all_experts, int unit_real, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || top <= 0) return NI_ERR_BAD_ARGUMENT;
    if (d > 12000) return NI_ERR_UNSUPPORTED_SIZE;
    const int threads = d >= 1024 ? 256 : 128;
    const size_t smem = (size_t)d * sizeof(float);
    if (top <= RT_MAX_EXPERTS && dtype == NI_DTYPE_BF16 && d % 8 == 0) {
        combine_add_normed_vec_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(
            (const __nv_bfloat16*)z, (const __nv_bfloat16*)x, ids, weights, row_of_pair, h, gain, eps, d, top, n_real, all_experts, unit_real);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (top <= RT_MAX_EXPERTS && dtype == NI_DTYPE_F32 && d % 4 == 0) {
        combine_add_normed_vec_kernel<float><<<n_tokens, threads, smem, stream>>>(
            (const float*)z, (const float*)x, ids, weights, row_of_pair, h, gain, eps, d, top, n_real, all_experts, unit_real);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (dtype == NI_DTYPE_F32)
        combine_add_normed_kernel<float><<<n_tokens, threads, smem, stream>>>((const float*)z, (const float*)x, ids, weights,
                                                                             row_of_pair, h, gain, eps, d, top, n_real, all_experts, unit_real);
    else if (dtype == NI_DTYPE_BF16)
        combine_add_normed_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(
            (const __nv_bfloat16*)z, (const __nv_bfloat16*)x, ids, weights, row_of_pair, h, gain, eps, d, top, n_real, all_experts, unit_real);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_route_combine(const void* z, const void* x, int dtype, const int* ids, const float* weights,
                               const int* row_of_pair, float* y, int n_tokens, int d, int top, int n_real,
                               int all_experts, int unit_real, int accumulate, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || top <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == NI_DTYPE_F32)
        combine_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)z, (const float*)x, ids, weights, row_of_pair, y,
                                                               d, top, n_real, all_experts, unit_real, accumulate);
    else if (dtype == NI_DTYPE_BF16)
        combine_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>((const __nv_bfloat16*)z, (const __nv_bfloat16*)x, ids,
                                                                       weights, row_of_pair, y, d, top, n_real, all_experts,
                                                                       unit_real, accumulate);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
