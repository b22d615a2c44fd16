// Latent attention keeps ONE compressed vector per token: c = RMSNorm(W_dkv x) (plain weight).
// Keys and values of every head are products of c (k = W_uk c, v = W_uv c), so the attention
// itself can run over the latents: the query is carried into the latent space (W_uk^T q, per
// head), scores and the weighted sum are taken over the pages of c, and the result leaves
// through W_uv.  These are the two small kernels around that: the normed write of a step's
// latents into their pages, and the per-head output gate.
#include "common.cuh"

// pages[page, in_page, :] = x / sqrt(mean(x^2) + eps) * weight, x = columns [col0, col0 + R) of proj[t].
// pages: [P, page_size, R]; the token's page comes from its request's block table.
template <typename T>
__global__ void latent_norm_write_kernel(const T* __restrict__ proj, int ld, int col0, const float* __restrict__ weight,
                                         float eps, T* __restrict__ pages, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                         int bt_stride, int R, int page_size) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    const T* x = proj + (size_t)t * ld + col0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = ni_to_float(x[i]);
        ss += v * v;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * R;
    for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = ni_from_float<T>(ni_to_float(x[i]) * inv * weight[i]);
}

NI_EXPORT int ni_latent_norm_write(const void* proj, int dtype, int ld, int col0, const float* weight, float eps,
                                   void* pages, const int* positions, const int* seq_of_token, const int* block_table,
                                   int bt_stride, int n_tokens, int R, int page_size, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (R <= 0 || page_size <= 0 || col0 < 0 || col0 + R > ld) return NI_ERR_BAD_ARGUMENT;
    const int threads = R >= 1024 ? 256 : 128;
#define LAUNCH(T)                                                                                              \
    latent_norm_write_kernel<T><<<n_tokens, threads, 0, stream>>>((const T*)proj, ld, col0, weight, eps, (T*)pages, \
                                                                  positions, seq_of_token, block_table, bt_stride, R, page_size)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

// x[t, h, :] *= sigmoid(proj[t, col0 + h]) * scale;  x [T, H, V]
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ proj, int ld, int col0, int n_tokens, int H,
                                 int V, float scale) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_tokens * H * V) return;
    const long long th = idx / V;
    const int t = (int)(th / H), h = (int)(th - (long long)t * H);
    const float g = scale / (1.0f + expf(-ni_to_float(proj[(size_t)t * ld + col0 + h])));
    x[idx] = ni_from_float<T>(ni_to_float(x[idx]) * g);
}

// The same, 16 bytes per thread (head sizes that are multiples of 8 bfloat16 or 4 float values).
template <typename T>
__global__ void head_gate_vec_kernel(T* __restrict__ x, const T* __restrict__ proj, int ld, int col0, long long n_vec, int H,
                                     int V, float scale) {
    constexpr int N = NiVec16<T>::N;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vec) return;
    const long long th = i / (V / N);
    const int t = (int)(th / H), h = (int)(th - (long long)t * H);
    const float g = scale / (1.0f + expf(-ni_to_float(proj[(size_t)t * ld + col0 + h])));
    float v[N];
    NiVec16<T>::load(x + i * N, v);
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] *= g;
    NiVec16<T>::store(x + i * N, v);
}

// scale: one more factor on every gate (1: none) - a mixer whose output is weighted before it is added to another's.
NI_EXPORT int ni_head_gate(void* x, int dtype, const void* proj, int ld, int col0, int n_tokens, int H, int V, float scale,
                           cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (H <= 0 || V <= 0 || col0 < 0 || col0 + H > ld) return NI_ERR_BAD_ARGUMENT;
    const long long blocks = ((long long)n_tokens * H * V + 255) / 256;
    if (blocks > 2147483647LL) return NI_ERR_UNSUPPORTED_SIZE;
    if (dtype == NI_DTYPE_BF16 && V % 8 == 0) {
        const long long nv = (long long)n_tokens * H * V / 8;
        head_gate_vec_kernel<__nv_bfloat16><<<(int)((nv + 255) / 256), 256, 0, stream>>>(
            (__nv_bfloat16*)x, (const __nv_bfloat16*)proj, ld, col0, nv, H, V, scale);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (dtype == NI_DTYPE_F32 && V % 4 == 0) {
        const long long nv = (long long)n_tokens * H * V / 4;
        head_gate_vec_kernel<float><<<(int)((nv + 255) / 256), 256, 0, stream>>>((float*)x, (const float*)proj, ld, col0, nv, H, V, scale);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (dtype == NI_DTYPE_F32)
        head_gate_kernel<float><<<(int)blocks, 256, 0, stream>>>((float*)x, (const float*)proj, ld, col0, n_tokens, H, V, scale);
    else if (dtype == NI_DTYPE_BF16)
        head_gate_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)proj, ld,
                                                                        col0, n_tokens, H, V, scale);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}


// A latent cache row with a rotated key part: beside c = RMSNorm(first R columns) * weight a token keeps rot_dim more
// numbers - one key part that all heads share and that is rotated by position - so a page row is [c | rot(k_r)], R +
// rot_dim wide.  The same launch rotates the last rot_dim dimensions of every head of q [T, H (R + rot_dim)] in place
// (queries that were carried into the latent space, with their rotated part behind).  Rotation: the angle
// float(position) * inv_freq[i] turns the pair (2i, 2i + 1) (`interleaved`) or (i, i + rot_dim / 2).
// One block per token.
template <typename T>
__global__ void latent_rope_write_kernel(const T* __restrict__ proj, int ld, int col0, const float* __restrict__ weight,
                                         float eps, T* __restrict__ pages, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                         int bt_stride, int R, int rot_dim, int page_size, const float* __restrict__ inv_freq,
                                         int interleaved, T* __restrict__ q, int H) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float cs[];          // [rot_dim]: cosines, then sines
    const int t = blockIdx.x, half = rot_dim >> 1, W = R + rot_dim;
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    const T* x = proj + (size_t)t * ld + col0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = ni_to_float(x[i]);
        ss += v * v;
    }
    ss = ni_block_sum(ss, scratch);                      // (its barriers also publish cs)
    const float inv = 1.0f / sqrtf(ss / (float)R + eps);
    if (pages) {
        const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
        T* dst = pages + ((size_t)page * page_size + pos % page_size) * W;
        for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = ni_from_float<T>(ni_to_float(x[i]) * inv * weight[i]);
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
            const float u = ni_to_float(x[R + a]), v = ni_to_float(x[R + b]);
            dst[R + a] = ni_from_float<T>(u * cs[i] - v * cs[half + i]);
            dst[R + b] = ni_from_float<T>(v * cs[i] + u * cs[half + i]);
        }
    }
    for (int j = threadIdx.x; j < H * half; j += blockDim.x) {
        const int head = j / half, i = j - head * half;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        T* qr = q + ((size_t)t * H + head) * W + R;
        const float u = ni_to_float(qr[a]), v = ni_to_float(qr[b]);
        qr[a] = ni_from_float<T>(u * cs[i] - v * cs[half + i]);
        qr[b] = ni_from_float<T>(v * cs[i] + u * cs[half + i]);
    }
}

// proj columns [col0, col0 + R + rot_dim): the latent, then the shared key part; pages [P, page_size, R + rot_dim] (null:
// nothing is written); q [T, H (R + rot_dim)].
NI_EXPORT int ni_latent_rope_write(const void* proj, int dtype, int ld, int col0, const float* weight, float eps,
                                   void* pages, const int* positions, const int* seq_of_token, const int* block_table,
                                   int bt_stride, int n_tokens, int R, int rot_dim, int page_size, const float* inv_freq,
                                   int interleaved, void* q, int H, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (R <= 0 || rot_dim < 0 || (rot_dim & 1) || page_size <= 0 || col0 < 0 || col0 + R + rot_dim > ld || H <= 0)
        return NI_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(rot_dim > 0 ? rot_dim : 1) * sizeof(float);
    if (smem > 48 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
    const int threads = R >= 1024 ? 256 : 128;
#define LAUNCH(T)                                                                                                     \
    latent_rope_write_kernel<T><<<n_tokens, threads, smem, stream>>>((const T*)proj, ld, col0, weight, eps, (T*)pages, \
                                                                     positions, seq_of_token, block_table, bt_stride, R, \
                                                                     rot_dim, page_size, inv_freq, interleaved, (T*)q, H)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
