// Row-wise kernels that several designs share: an embedding with a sinusoidal position vector,
// a cast of the FP32 residual stream to the compute dtype, a normed addition into the stream, the
// PolyNorm activation, and a gate multiplied by a per-token table row.
//
// All statistics, angles and activation arguments are FP32; inputs and outputs are FP32 or
// bfloat16 as their tensors say.  One block per row, sums in a fixed order, so a row's result
// never depends on what else is in the step.
#include "common.cuh"

// out[t, 2i] = table[tok, 2i] + sin(p * f_i), out[t, 2i+1] = table[tok, 2i+1] + cos(p * f_i),
// with p = positions[t] and f_i = inv_freq[i] (computed on the host, rounded once to FP32).
template <typename T>
__global__ void embedding_sinusoid_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                          const T* __restrict__ table, const float* __restrict__ inv_freq,
                                          float* __restrict__ out, int d, int vocab) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    const T* row = table + (size_t)(ok ? tok : 0) * d;
    const float p = (float)positions[t];
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float ang = __fmul_rn(p, inv_freq[i >> 1]);
        const float pe = (i & 1) ? cosf(ang) : sinf(ang);
        o[i] = (ok ? ni_to_float(row[i]) : 0.f) + pe;
    }
}

NI_EXPORT int ni_embedding_sinusoid(const int* tokens, const int* positions, const void* table, int table_dtype,
                                    const float* inv_freq, float* out, int n_tokens, int d, int vocab,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == NI_DTYPE_F32)
        embedding_sinusoid_kernel<float><<<n_tokens, threads, 0, stream>>>(tokens, positions, (const float*)table,
                                                                           inv_freq, out, d, vocab);
    else if (table_dtype == NI_DTYPE_BF16)
        embedding_sinusoid_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            tokens, positions, (const __nv_bfloat16*)table, inv_freq, out, d, vocab);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out = bfloat16(x), element by element (x FP32).
__global__ void cast_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(x[i]);
}

// The same, eight numbers per thread (n a multiple of 8, both on 16 bytes).
__global__ void cast_bf16_vec_kernel(const float4* __restrict__ x, uint4* __restrict__ out, long long n8) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float4 a = x[2 * i], b = x[2 * i + 1];
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    const __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&p0); o.y = *reinterpret_cast<const uint32_t*>(&p1);
    o.z = *reinterpret_cast<const uint32_t*>(&p2); o.w = *reinterpret_cast<const uint32_t*>(&p3);
    out[i] = o;
}

NI_EXPORT int ni_cast_bf16(const float* x, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return NI_OK;
    if (n % 8 == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(out)) & 15) == 0) {
        const long long n8 = n / 8, vb = (n8 + 255) / 256;
        if (vb > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
        cast_bf16_vec_kernel<<<(int)vb, 256, 0, stream>>>((const float4*)x, (uint4*)out, n8);
        NI_RETURN_LAUNCH_STATUS();
    }
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    cast_bf16_kernel<<<(int)blocks, 256, 0, stream>>>(x, (__nv_bfloat16*)out, n);
    NI_RETURN_LAUNCH_STATUS();
}

// h[t, :] += z / sqrt(mean(z^2) + eps) * weight with z = y[t, :] (+ bias, FP32 [d], where one is given: a product's
// bias that its kernel did not add)
// `rounded` (bfloat16 [rows, d], or null): the updated row once more in bfloat16 - what the next sublayer reads when it
// takes the stream itself.
template <typename T>
__global__ void add_normed_kernel(float* __restrict__ h, const T* __restrict__ y, const float* __restrict__ weight,
                                  float eps, int d, const float* __restrict__ bias, __nv_bfloat16* __restrict__ rounded) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* yr = y + (size_t)t * d;
    float* hr = h + (size_t)t * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = ni_to_float(yr[i]) + (bias ? bias[i] : 0.f);
        ss += v * v;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = hr[i] + (ni_to_float(yr[i]) + (bias ? bias[i] : 0.f)) * inv * weight[i];
        hr[i] = v;
        if (rounded) rounded[(size_t)t * d + i] = __float2bfloat16_rn(v);
    }
}

// The same for FP32 y whose width is a multiple of 4, up to 4,096: the row stays in the block's registers between
// the sum of squares and the addition, and moves in 16-byte pieces.
__global__ void __launch_bounds__(256)
add_normed_f32_vec_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ weight, float eps,
                          int d, const float* __restrict__ bias, __nv_bfloat16* __restrict__ rounded) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * d);
    float4* hr = reinterpret_cast<float4*>(h + (size_t)t * d);
    const float4* wr = reinterpret_cast<const float4*>(weight);
    const int n4 = d >> 2;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = threadIdx.x + 256 * r;
        v[r] = i < n4 ? yr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias && i < n4) {
            const float4 b = reinterpret_cast<const float4*>(bias)[i];
            v[r].x += b.x; v[r].y += b.y; v[r].z += b.z; v[r].w += b.w;
        }
        ss += v[r].x * v[r].x + v[r].y * v[r].y + v[r].z * v[r].z + v[r].w * v[r].w;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int i = threadIdx.x + 256 * r;
        if (i < n4) {
            float4 a = hr[i];
            const float4 g = wr[i];
            a.x += v[r].x * inv * g.x;
            a.y += v[r].y * inv * g.y;
            a.z += v[r].z * inv * g.z;
            a.w += v[r].w * inv * g.w;
            hr[i] = a;
            if (rounded) {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
                uint2 packed;
                packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(rounded + (size_t)t * d)[i] = packed;
            }
        }
    }
}

NI_EXPORT int ni_add_normed(float* h, const void* y, int y_dtype, const float* weight, float eps, int n_rows, int d,
                            const float* bias, void* rounded, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (d <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    __nv_bfloat16* rb = (__nv_bfloat16*)rounded;
    if (y_dtype == NI_DTYPE_F32 && d % 4 == 0 && d <= 4096 && d >= 512 && (reinterpret_cast<size_t>(bias) & 15) == 0 &&
        (reinterpret_cast<size_t>(rounded) & 7) == 0)
        add_normed_f32_vec_kernel<<<n_rows, 256, 0, stream>>>(h, (const float*)y, weight, eps, d, bias, rb);
    else if (y_dtype == NI_DTYPE_F32)
        add_normed_kernel<float><<<n_rows, threads, 0, stream>>>(h, (const float*)y, weight, eps, d, bias, rb);
    else if (y_dtype == NI_DTYPE_BF16)
        add_normed_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(h, (const __nv_bfloat16*)y, weight, eps, d, bias, rb);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// PolyNorm: out = c1 R(z) + c2 R(z * z) + c3 R(z * z * z) + c0: the first three powers of every value, each
// power divided by its own root mean square over the row (eps under the root).  coef = {c1, c2, c3, c0}.
template <typename T>
__global__ void polynorm_kernel(const T* __restrict__ z, const float* __restrict__ coef, float eps,
                                T* __restrict__ out, int n) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* zr = z + (size_t)t * n;
    T* o = out + (size_t)t * n;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = ni_to_float(zr[i]);
        const float v2 = v * v;
        s1 += v2;
        s2 += v2 * v2;
        s3 += (v2 * v) * (v2 * v);
    }
    s1 = ni_block_sum(s1, scratch);
    s2 = ni_block_sum(s2, scratch);
    s3 = ni_block_sum(s3, scratch);
    const float r1 = coef[0] / sqrtf(s1 / (float)n + eps);
    const float r2 = coef[1] / sqrtf(s2 / (float)n + eps);
    const float r3 = coef[2] / sqrtf(s3 / (float)n + eps);
    const float e = coef[3];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = ni_to_float(zr[i]);
        const float v2 = v * v;
        o[i] = ni_from_float<T>(v * r1 + v2 * r2 + (v2 * v) * r3 + e);
    }
}

// The same for bfloat16 rows whose length is a multiple of 8: 16-byte accesses, the three sums reduced together.
// Each thread's elements and the order of every sum differ from the kernel above only in how the row is dealt
// out, which depends on the row's length alone, never on the number of rows.
__global__ void __launch_bounds__(256)
polynorm_bf16_vec_kernel(const __nv_bfloat16* __restrict__ z, const float* __restrict__ coef, float eps,
                         __nv_bfloat16* __restrict__ out, int n) {
    __shared__ float red[3][8];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4* zr = reinterpret_cast<const uint4*>(z + (size_t)t * n);
    uint4* orow = reinterpret_cast<uint4*>(out + (size_t)t * n);
    const int n8 = n >> 3;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < n8; i += 256) {
        const uint4 pk = zr[i];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            const float a2 = f.x * f.x, b2 = f.y * f.y;
            s1 += a2 + b2;
            s2 += a2 * a2 + b2 * b2;
            s3 += (a2 * f.x) * (a2 * f.x) + (b2 * f.y) * (b2 * f.y);
        }
    }
    s1 = ni_warp_sum(s1); s2 = ni_warp_sum(s2); s3 = ni_warp_sum(s3);
    if (lane == 0) { red[0][warp] = s1; red[1][warp] = s2; red[2][warp] = s3; }
    __syncthreads();
    s1 = s2 = s3 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { s1 += red[0][w]; s2 += red[1][w]; s3 += red[2][w]; }
    const float r1 = coef[0] / sqrtf(s1 / (float)n + eps);
    const float r2 = coef[1] / sqrtf(s2 / (float)n + eps);
    const float r3 = coef[2] / sqrtf(s3 / (float)n + eps);
    const float e = coef[3];
    for (int i = threadIdx.x; i < n8; i += 256) {
        uint4 pk = zr[i];
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h2[j]);
            const float a2 = f.x * f.x, b2 = f.y * f.y;
            h2[j] = __floats2bfloat162_rn(f.x * r1 + a2 * r2 + (a2 * f.x) * r3 + e, f.y * r1 + b2 * r2 + (b2 * f.y) * r3 + e);
        }
        orow[i] = pk;
    }
}

NI_EXPORT int ni_polynorm(const void* z, int dtype, const float* coef, float eps, void* out, int n_rows, int n,
                          cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (n <= 0) return NI_ERR_BAD_ARGUMENT;
    if (dtype == NI_DTYPE_BF16 && n % 8 == 0 && ((uintptr_t)z & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        polynorm_bf16_vec_kernel<<<n_rows, 256, 0, stream>>>((const __nv_bfloat16*)z, coef, eps, (__nv_bfloat16*)out, n);
        NI_RETURN_LAUNCH_STATUS();
    }
    const int threads = n >= 2048 ? 512 : (n >= 512 ? 256 : 128);
    if (dtype == NI_DTYPE_F32)
        polynorm_kernel<float><<<n_rows, threads, 0, stream>>>((const float*)z, coef, eps, (float*)out, n);
    else if (dtype == NI_DTYPE_BF16)
        polynorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>((const __nv_bfloat16*)z, coef, eps,
                                                                      (__nv_bfloat16*)out, n);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out[t, j] = gelu_tanh(gate[t, j]) * table[tokens[t], first + j],  j < n; the table has `stride` columns.
// The gate is the tanh form of GELU: z / 2 * (1 + tanh(c * (z + 0.044715 z^3))) with c = sqrt(2 / pi).
template <typename T, typename TT>
__global__ void gelu_table_gate_kernel(const T* __restrict__ gate, const int* __restrict__ tokens,
                                       const TT* __restrict__ table, T* __restrict__ out, int n_rows, int n,
                                       int first, int stride, int vocab) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_rows * n) return;
    const int t = (int)(idx / n), j = (int)(idx - (long long)t * n);
    const int tok = tokens[t];
    const float e = (tok >= 0 && tok < vocab) ? ni_to_float(table[(size_t)tok * stride + first + j]) : 0.f;
    const float z = ni_to_float(gate[idx]);
    const float g = 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    out[idx] = ni_from_float<T>(g * e);
}

NI_EXPORT int ni_gelu_table_gate(const void* gate, int dtype, const int* tokens, const void* table, int table_dtype,
                                 void* out, int n_rows, int n, int first, int stride, int vocab, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return NI_OK;
    if (first < 0 || first + n > stride || vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    const long long blocks = ((long long)n_rows * n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
#define LAUNCH(T, TT)                                                                                          \
    gelu_table_gate_kernel<T, TT><<<(int)blocks, 256, 0, stream>>>((const T*)gate, tokens, (const TT*)table, \
                                                                   (T*)out, n_rows, n, first, stride, vocab)
    if (dtype == NI_DTYPE_F32 && table_dtype == NI_DTYPE_F32) LAUNCH(float, float);
    else if (dtype == NI_DTYPE_BF16 && table_dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

// h[t, :] += row[:] for every token (a learned vector that joins the stream); FP32.
template <typename T>
__global__ void add_row_kernel(float* __restrict__ h, const T* __restrict__ row, long long n, int d) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] += ni_to_float(row[i % d]);
}

NI_EXPORT int ni_add_row(float* h, const void* row, int row_dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (d <= 0) return NI_ERR_BAD_ARGUMENT;
    const long long n = (long long)n_rows * d, blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (row_dtype == NI_DTYPE_F32) add_row_kernel<float><<<(int)blocks, 256, 0, stream>>>(h, (const float*)row, n, d);
    else if (row_dtype == NI_DTYPE_BF16)
        add_row_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(h, (const __nv_bfloat16*)row, n, d);
    else return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// x *= factor, element by element (FP32: logits).
__global__ void scale_f32_kernel(float* __restrict__ x, float factor, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= factor;
}

NI_EXPORT int ni_scale_f32(float* x, float factor, long long n, cudaStream_t stream) {
    if (n <= 0) return NI_OK;
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    scale_f32_kernel<<<(int)blocks, 256, 0, stream>>>(x, factor, n);
    NI_RETURN_LAUNCH_STATUS();
}

// A gated unit with capped arguments: g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(slope * g) * (u + shift); gate_up = [gate | up] along the columns.  bias (FP32 [2 inter], gate
// then up, or null) joins gate and up before the limits.
template <typename T>
__global__ void capped_glu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long n, int inter,
                                  float limit, float slope, float shift, const float* __restrict__ row_scale,
                                  const float* __restrict__ bias) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / inter;
    const int c = (int)(i - t * inter);
    const T* row = gate_up + (size_t)t * 2 * inter;
    const float rs = row_scale ? row_scale[t] : 1.0f;
    const float g = fminf(ni_to_float(row[c]) * rs + (bias ? bias[c] : 0.f), limit);
    const float u = fminf(fmaxf(ni_to_float(row[inter + c]) * rs + (bias ? bias[inter + c] : 0.f), -limit), limit);
    out[i] = ni_from_float<T>(g / (1.0f + expf(-slope * g)) * (u + shift));
}

// The same, 16 bytes per thread (row widths that are multiples of 8 bfloat16 or 4 float values).
template <typename T>
__global__ void capped_glu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long n_vec, int inter,
                                      float limit, float slope, float shift, const float* __restrict__ row_scale,
                                      const float* __restrict__ bias) {
    constexpr int V = NiVec16<T>::N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const int per_row = inter / V;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row) * V;
    const T* row = gate_up + (size_t)t * 2 * inter;
    float g[V], u[V], o[V];
    NiVec16<T>::load(row + c, g);
    NiVec16<T>::load(row + inter + c, u);
    const float rs = row_scale ? row_scale[t] : 1.0f;
    float bg[V], bu[V];
#pragma unroll
    for (int k = 0; k < V; ++k) bg[k] = bu[k] = 0.f;
    if (bias) {                       // 16-byte loads where the two halves of the bias start on 16 bytes
        if ((inter & 3) == 0 && (reinterpret_cast<size_t>(bias) & 15) == 0) {
#pragma unroll
            for (int k = 0; k < V; k += 4) {
                const float4 a = *reinterpret_cast<const float4*>(bias + c + k), b = *reinterpret_cast<const float4*>(bias + inter + c + k);
                bg[k] = a.x; bg[k + 1] = a.y; bg[k + 2] = a.z; bg[k + 3] = a.w;
                bu[k] = b.x; bu[k + 1] = b.y; bu[k + 2] = b.z; bu[k + 3] = b.w;
            }
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k) { bg[k] = bias[c + k]; bu[k] = bias[inter + c + k]; }
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
        const float gg = fminf(g[k] * rs + bg[k], limit);
        const float uu = fminf(fmaxf(u[k] * rs + bu[k], -limit), limit);
        o[k] = gg / (1.0f + expf(-slope * gg)) * (uu + shift);
    }
    NiVec16<T>::store(out + (size_t)t * inter + c, o);
}

// row_scale (FP32 [rows], or null): the row's gate and up values are multiplied by it before the limits, which is
// what a unit computes when its INPUT was multiplied by that number (both products are linear in the input).
NI_EXPORT int ni_capped_glu(const void* gate_up, void* out, int dtype, int n_rows, int inter, float limit, float slope,
                            float shift, const float* row_scale, const float* bias, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (inter <= 0) return NI_ERR_BAD_ARGUMENT;
    const long long n = (long long)n_rows * inter, blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (dtype == NI_DTYPE_BF16 && inter % 8 == 0) {
        const long long nv = n / 8;
        capped_glu_vec_kernel<__nv_bfloat16><<<(int)((nv + 255) / 256), 256, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, nv, inter, limit, slope, shift, row_scale, bias);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (dtype == NI_DTYPE_F32 && inter % 4 == 0) {
        const long long nv = n / 4;
        capped_glu_vec_kernel<float><<<(int)((nv + 255) / 256), 256, 0, stream>>>((const float*)gate_up, (float*)out, nv, inter,
                                                                                limit, slope, shift, row_scale, bias);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (dtype == NI_DTYPE_F32)
        capped_glu_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, n, inter, limit, slope, shift, row_scale, bias);
    else if (dtype == NI_DTYPE_BF16)
        capped_glu_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, n,
                                                                         inter, limit, slope, shift, row_scale, bias);
    else return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out[t, :] = table[tokens[t], :] * scale as FP32 (an id out of range writes zeros).
template <typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float scale,
                                        float* __restrict__ out, int d, int vocab) {
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    const T* row = table + (size_t)(ok ? tok : 0) * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? ni_to_float(row[i]) * scale : 0.f;
}

NI_EXPORT int ni_embedding_scaled(const int* tokens, const void* table, int table_dtype, float scale, float* out,
                                  int n_tokens, int d, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || vocab <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (table_dtype == NI_DTYPE_F32)
        embedding_scaled_kernel<float><<<n_tokens, threads, 0, stream>>>(tokens, (const float*)table, scale, out, d, vocab);
    else if (table_dtype == NI_DTYPE_BF16)
        embedding_scaled_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(tokens, (const __nv_bfloat16*)table, scale,
                                                                                out, d, vocab);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out[t, :] = [a[t, :] | b[t, :]] in the activations' type: two FP32 streams side by side as one product's input.
template <typename T>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int d) {
    const int t = blockIdx.x;
    const float* ar = a + (size_t)t * d;
    const float* br = b + (size_t)t * d;
    T* o = out + (size_t)t * 2 * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        o[i] = ni_from_float<T>(ar[i]);
        o[d + i] = ni_from_float<T>(br[i]);
    }
}

NI_EXPORT int ni_concat_cast(const float* a, const float* b, void* out, int dtype, int n_rows, int d, cudaStream_t stream) {
    if (n_rows <= 0) return NI_OK;
    if (d <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == NI_DTYPE_F32) concat_cast_kernel<float><<<n_rows, threads, 0, stream>>>(a, b, (float*)out, d);
    else if (dtype == NI_DTYPE_BF16) concat_cast_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(a, b, (__nv_bfloat16*)out, d);
    else return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out = max(z, 0)^2, element by element, FP32 inside.
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ z, T* __restrict__ out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = fmaxf(ni_to_float(z[i]), 0.f);
    out[i] = ni_from_float<T>(v * v);
}

// The same, 16 bytes per thread (counts that are multiples of 8 bfloat16 or 4 float values).
template <typename T>
__global__ void relu_squared_vec_kernel(const T* __restrict__ z, T* __restrict__ out, long long n_vec) {
    constexpr int V = NiVec16<T>::N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    float v[V];
    NiVec16<T>::load(z + i * V, v);
#pragma unroll
    for (int k = 0; k < V; ++k) {
        const float r = fmaxf(v[k], 0.f);
        v[k] = r * r;
    }
    NiVec16<T>::store(out + i * V, v);
}

NI_EXPORT int ni_relu_squared(const void* z, void* out, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return NI_OK;
    const int per = dtype == NI_DTYPE_BF16 ? 8 : 4;
    if (dtype != NI_DTYPE_BF16 && dtype != NI_DTYPE_F32) return NI_ERR_BAD_ARGUMENT;
    if (n % per == 0) {
        const long long nv = n / per, blocks = (nv + 255) / 256;
        if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
        if (dtype == NI_DTYPE_BF16)
            relu_squared_vec_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)z, (__nv_bfloat16*)out, nv);
        else
            relu_squared_vec_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)z, (float*)out, nv);
        NI_RETURN_LAUNCH_STATUS();
    }
    const long long blocks = (n + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (dtype == NI_DTYPE_BF16)
        relu_squared_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)z, (__nv_bfloat16*)out, n);
    else
        relu_squared_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)z, (float*)out, n);
    NI_RETURN_LAUNCH_STATUS();
}


// An embedding with a second table that is addressed by a hash of the token and the one before it:
//   out[t, :] = table[token, :] + pairs[r, :],   r = (previous * mul_prev + token * mul_cur) mod buckets,
// and r = buckets (the table's last row) for a sequence's first token.  The token before a step's first one is part of
// the request's state: last[slot] holds the last token of the step before and is set to this step's last one by the
// block that read it (the block of the request's first token in the step), so a step may be cut anywhere and a
// captured step finds everything on the device.  One block per token; FP32 sum.
template <typename T>
__global__ void embedding_pairs_kernel(const int* __restrict__ tokens, const T* __restrict__ table, const T* __restrict__ pairs,
                                       float* __restrict__ out, int d, int vocab, int buckets, int mul_prev, int mul_cur,
                                       const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                       const int* __restrict__ cu_q, const int* __restrict__ slots, int* __restrict__ last) {
    __shared__ int s_row;
    const int t = blockIdx.x;
    const int tok = tokens[t];
    if (threadIdx.x == 0) {
        const int seq = seq_of_token[t], first = cu_q[seq];
        int prev = 0;
        if (t > first) {
            prev = tokens[t - 1];
        } else {
            int* mine = last + slots[seq];
            prev = *mine;
            *mine = tokens[cu_q[seq + 1] - 1];
        }
        s_row = positions[t] == 0 ? buckets
                                  : (int)(((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets);
    }
    __syncthreads();
    const bool ok = tok >= 0 && tok < vocab;
    const int r = s_row < 0 ? s_row + buckets : s_row;
    const T* row = table + (size_t)(ok ? tok : 0) * d;
    const T* pr = pairs + (size_t)r * d;
    float* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? ni_to_float(row[i]) + ni_to_float(pr[i]) : 0.f;
}

// table [vocab, d] and pairs [buckets + 1, d] of one type; last int32 [slots].
NI_EXPORT int ni_embedding_pairs(const int* tokens, const void* table, const void* pairs, int dtype, float* out, int n_tokens,
                                 int d, int vocab, int buckets, int mul_prev, int mul_cur, const int* positions,
                                 const int* seq_of_token, const int* cu_q, const int* slots, int* last, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (d <= 0 || vocab <= 0 || buckets <= 0) return NI_ERR_BAD_ARGUMENT;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == NI_DTYPE_F32)
        embedding_pairs_kernel<float><<<n_tokens, threads, 0, stream>>>(tokens, (const float*)table, (const float*)pairs, out, d,
                                                                        vocab, buckets, mul_prev, mul_cur, positions,
                                                                        seq_of_token, cu_q, slots, last);
    else if (dtype == NI_DTYPE_BF16)
        embedding_pairs_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
            tokens, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pairs, out, d, vocab, buckets, mul_prev, mul_cur,
            positions, seq_of_token, cu_q, slots, last);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// out = sa * a + sb * b, element by element (FP32; out may be a or b).
__global__ void weighted_sum_kernel(const float* a, float sa, const float* b, float sb, float* out, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = sa * a[i] + sb * b[i];
}

// The same, four numbers per thread (n a multiple of 4, all three on 16 bytes).
__global__ void weighted_sum_vec_kernel(const float4* a, float sa, const float4* b, float sb, float4* out, long long n4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 x = a[i], y = b[i];
    out[i] = make_float4(sa * x.x + sb * y.x, sa * x.y + sb * y.y, sa * x.z + sb * y.z, sa * x.w + sb * y.w);
}

NI_EXPORT int ni_weighted_sum(const float* a, float sa, const float* b, float sb, float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return NI_OK;
    const bool wide = n % 4 == 0 && ((reinterpret_cast<size_t>(a) | reinterpret_cast<size_t>(b) | reinterpret_cast<size_t>(out)) & 15) == 0;
    const long long items = wide ? n / 4 : n, blocks = (items + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (wide)
        weighted_sum_vec_kernel<<<(int)blocks, 256, 0, stream>>>((const float4*)a, sa, (const float4*)b, sb, (float4*)out, items);
    else
        weighted_sum_kernel<<<(int)blocks, 256, 0, stream>>>(a, sa, b, sb, out, n);
    NI_RETURN_LAUNCH_STATUS();
}
