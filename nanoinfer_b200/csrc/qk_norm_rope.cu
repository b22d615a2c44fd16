// What lies between the fused q | k | v projection and the attention of a mixer whose queries and keys are
// normed as a whole: per token, in FP32 whatever the tensors' type,
//
//   q, k, v  += bias                         (optional; one FP32 vector over the projection's columns)
//   q <- q / sqrt(mean(q^2) + eps) * gain    over ALL H * D query values at once, and likewise the G * D key
//                                            values (optional; gains FP32 [H D] and [G D])
//   rotation of the first `rotary_dim` dimensions of every head of q and k, dimension i paired with
//            i + rotary_dim / 2:  (u, v) -> (u c - v s, v c + u s),  c = m cos(a), s = m sin(a),
//            a = float(position) * inv_freq[i]  (m = `magnitude`: an encoding that also scales what it rotates)
//   (optional, `head_unit`) every head of q and of k divided by its own root mean square over D, eps inside the
//            root, no weight - after the rotation
//   q -> q_out [T, H D];  k -> key pages [P, G, page, D];  v -> value pages [P, G, page, V]
//
// One block per token.  The row's queries and keys are widened once into shared memory, where the two sums of
// squares and the partner of every rotated dimension are found; the angles' cosines and sines are computed
// once per token and shared by all heads.
#include "common.cuh"

// The heads' own norms: vals [(H + G) D] in shared memory holds the token's finished queries and keys; a warp takes
// a head at a time, divides it by its root mean square and writes it out (a key only where there are pages).
template <typename T>
__device__ __forceinline__ void qk_head_unit_write(const float* __restrict__ vals, float eps, T* __restrict__ q_row,
                                                   T* __restrict__ kdst, int H, int G, int D, int page_size) {
    __syncthreads();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int head = threadIdx.x >> 5; head < H + G; head += warps) {
        const float* x = vals + (size_t)head * D;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss = fmaf(x[d], x[d], ss);
        ss = ni_warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)D + eps);
        T* dst = head < H ? q_row + (size_t)head * D : (kdst ? kdst + (size_t)(head - H) * page_size * D : nullptr);
        if (dst)
            for (int d = lane; d < D; d += 32) dst[d] = ni_from_float<T>(x[d] * inv);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const T* __restrict__ qkv, int ld, const float* __restrict__ bias,
                    const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                    const int* __restrict__ block_table, int bt_stride, const float* __restrict__ inv_freq,
                    float magnitude, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                    int H, int G, int D, int V, int rotary_dim, int page_size, int head_unit) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float scratch[32];
    const int nq = H * D, nk = G * D, nv = G * V, half = rotary_dim >> 1;
    float* row = sm;                 // [nq + nk]: queries, then keys, bias added
    float* cs = sm + nq + nk;        // [2 half]: m cos, then m sin
    const int t = blockIdx.x;
    const T* x = qkv + (size_t)t * ld;
    const int pos = positions[t];
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const float v = ni_to_float(x[i]) + (bias ? bias[i] : 0.f);
        row[i] = v;
        if (i < nq) sq += v * v; else sk += v * v;
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c * magnitude;
        cs[half + i] = s * magnitude;
    }
    sq = ni_block_sum(sq, scratch);
    sk = ni_block_sum(sk, scratch);          // (its barriers also publish row and cs)
    const float inv_q = q_gain ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f;
    const float inv_k = k_gain ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.0f;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages) {
        const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
        const int in_page = pos % page_size;
        kdst = k_pages + ((size_t)page * G * page_size + in_page) * D;           // head g: + g * page_size * D
        vdst = v_pages + ((size_t)page * G * page_size + in_page) * V;
    }
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const bool is_q = i < nq;
        const int e = is_q ? i : i - nq;
        const int head = e / D, dim = e - head * D;
        const float* gain = is_q ? q_gain : k_gain;
        const float inv = is_q ? inv_q : inv_k;
        float a = row[i] * inv * (gain ? gain[e] : 1.0f);
        if (dim < rotary_dim) {
            const bool first = dim < half;
            const int other = first ? i + half : i - half, oe = first ? e + half : e - half;
            const float b = row[other] * inv * (gain ? gain[oe] : 1.0f);
            const int f = first ? dim : dim - half;
            a = first ? a * cs[f] - b * cs[half + f] : a * cs[f] + b * cs[half + f];
        }
        if (head_unit) cs[rotary_dim + i] = a;            // kept for the heads' own norms below
        else if (is_q) q_out[(size_t)t * nq + e] = ni_from_float<T>(a);
        else if (kdst) kdst[(size_t)head * page_size * D + dim] = ni_from_float<T>(a);
    }
    if (head_unit) qk_head_unit_write<T>(cs + rotary_dim, eps, q_out + (size_t)t * nq, kdst, H, G, D, page_size);
    if (vdst) {
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            const int head = i / V, dim = i - head * V;
            const float v = ni_to_float(x[nq + nk + i]) + (bias ? bias[nq + nk + i] : 0.f);
            vdst[(size_t)head * page_size * V + dim] = ni_from_float<T>(v);
        }
    }
}

// The same with 16 bytes per load and store: a thread owns VEC neighbouring dimensions (8 bfloat16 or 4 floats).
// For sizes whose heads, rotated halves and rows all start on 16 bytes (the launcher checks).
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_vec_kernel(const T* __restrict__ qkv, int ld, const float* __restrict__ bias,
                        const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ block_table, int bt_stride, const float* __restrict__ inv_freq,
                        float magnitude, T* __restrict__ q_out, T* __restrict__ k_pages, T* __restrict__ v_pages,
                        int H, int G, int D, int V, int rotary_dim, int page_size, int head_unit) {
    constexpr int VEC = 16 / sizeof(T);
    extern __shared__ __align__(16) float sm[];
    __shared__ float scratch[32];
    const int nq = H * D, nk = G * D, nv = G * V, half = rotary_dim >> 1;
    float* row = sm;                 // [nq + nk]: queries, then keys, bias added
    float* cs = sm + nq + nk;        // [2 half]: m cos, then m sin
    const int t = blockIdx.x;
    const T* x = qkv + (size_t)t * ld;
    const int pos = positions[t];
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x * VEC; i < nq + nk; i += blockDim.x * VEC) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + i);
        const T* e = reinterpret_cast<const T*>(&raw);
        float v[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[k] = ni_to_float(e[k]);
        if (bias) {
#pragma unroll
            for (int k = 0; k < VEC; k += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(bias + i + k);
                v[k] += b4.x; v[k + 1] += b4.y; v[k + 2] += b4.z; v[k + 3] += b4.w;
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VEC; ++k) ss = fmaf(v[k], v[k], ss);
        if (i < nq) sq += ss; else sk += ss;
#pragma unroll
        for (int k = 0; k < VEC; k += 4) *reinterpret_cast<float4*>(row + i + k) = make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]);
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[i] = c * magnitude;
        cs[half + i] = s * magnitude;
    }
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (k_pages) {
        const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
        const int in_page = pos % page_size;
        kdst = k_pages + ((size_t)page * G * page_size + in_page) * D;           // head g: + g * page_size * D
        vdst = v_pages + ((size_t)page * G * page_size + in_page) * V;
    }
    if (vdst) {                               // the values do not wait for the sums
        for (int i = threadIdx.x * VEC; i < nv; i += blockDim.x * VEC) {
            const int head = i / V, dim = i - head * V;
            uint4 raw = *reinterpret_cast<const uint4*>(x + nq + nk + i);
            if (bias) {
                T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
                for (int k = 0; k < VEC; ++k) e[k] = ni_from_float<T>(ni_to_float(e[k]) + bias[nq + nk + i + k]);
            }
            *reinterpret_cast<uint4*>(vdst + (size_t)head * page_size * V + dim) = raw;
        }
    }
    sq = ni_block_sum(sq, scratch);
    sk = ni_block_sum(sk, scratch);          // (its barriers also publish row and cs)
    const float inv_q = q_gain ? 1.0f / sqrtf(sq / (float)nq + eps) : 1.0f;
    const float inv_k = k_gain ? 1.0f / sqrtf(sk / (float)nk + eps) : 1.0f;
    for (int i = threadIdx.x * VEC; i < nq + nk; i += blockDim.x * VEC) {
        const bool is_q = i < nq;
        const int e = is_q ? i : i - nq;
        const int head = e / D, dim = e - head * D;
        const float* gain = is_q ? q_gain : k_gain;
        const float inv = is_q ? inv_q : inv_k;
        float a[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) a[k] = row[i + k] * inv * (gain ? gain[e + k] : 1.0f);
        if (dim < rotary_dim) {               // all VEC dimensions lie in the same half
            const bool first = dim < half;
            const int shift = first ? half : -half;
            const int f = first ? dim : dim - half;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                const float b = row[i + shift + k] * inv * (gain ? gain[e + shift + k] : 1.0f);
                a[k] = first ? a[k] * cs[f + k] - b * cs[half + f + k] : a[k] * cs[f + k] + b * cs[half + f + k];
            }
        }
        if (head_unit) {                       // kept for the heads' own norms below
#pragma unroll
            for (int k = 0; k < VEC; ++k) cs[rotary_dim + i + k] = a[k];
            continue;
        }
        uint4 packed;
        T* o = reinterpret_cast<T*>(&packed);
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = ni_from_float<T>(a[k]);
        if (is_q) *reinterpret_cast<uint4*>(q_out + (size_t)t * nq + e) = packed;
        else if (kdst) *reinterpret_cast<uint4*>(kdst + (size_t)head * page_size * D + dim) = packed;
    }
    if (head_unit) qk_head_unit_write<T>(cs + rotary_dim, eps, q_out + (size_t)t * nq, kdst, H, G, D, page_size);
}

// qkv [T, ld] with columns q (H D) | k (G D) | v (G V); bias FP32 [H D + G D + G V] or null; q_gain FP32 [H D] and
// k_gain FP32 [G D], or null for no norm; head_unit: the heads' own norms after the rotation; k_pages / v_pages null: nothing is written (a run that reads another's cache).
NI_EXPORT int ni_qk_norm_rope(const void* qkv, int dtype, int ld, const float* bias, const float* q_gain,
                              const float* k_gain, float eps, const int* positions, const int* seq_of_token,
                              const int* block_table, int bt_stride, const float* inv_freq, float magnitude, void* q_out,
                              void* k_pages, void* v_pages, int n_tokens, int H, int G, int D, int V, int rotary_dim,
                              int page_size, int head_unit, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (H <= 0 || G <= 0 || D <= 0 || V <= 0 || page_size <= 0 || rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) ||
        ld < (H + G) * D + G * V || (q_gain == nullptr) != (k_gain == nullptr))
        return NI_ERR_BAD_ARGUMENT;
    const size_t smem = ((size_t)(H + G) * D * (head_unit ? 2 : 1) + rotary_dim) * sizeof(float);
    if (smem > 200 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
    const int vec = dtype == NI_DTYPE_F32 ? 4 : 8;       // elements in 16 bytes
    const auto aligned = [](const void* p) { return (reinterpret_cast<size_t>(p) & 15) == 0; };
    const bool wide = D % vec == 0 && V % vec == 0 && (rotary_dim / 2) % vec == 0 && ld % vec == 0 && aligned(qkv) &&
                      aligned(q_out) && aligned(k_pages) && aligned(v_pages) && aligned(bias);
#define LAUNCH_VEC(T)                                                                                                \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(qk_norm_rope_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        qk_norm_rope_vec_kernel<T><<<n_tokens, threads, smem, stream>>>((const T*)qkv, ld, bias, q_gain, k_gain, eps, \
                                                                    positions, seq_of_token, block_table, bt_stride, \
                                                                    inv_freq, magnitude, (T*)q_out, (T*)k_pages,     \
                                                                    (T*)v_pages, H, G, D, V, rotary_dim, page_size, head_unit); \
    } while (0)
    if (wide && (dtype == NI_DTYPE_F32 || dtype == NI_DTYPE_BF16)) {
        const int work = ((H + G) * D + vec - 1) / vec;
        const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
        if (dtype == NI_DTYPE_F32) LAUNCH_VEC(float);
        else LAUNCH_VEC(__nv_bfloat16);
        NI_RETURN_LAUNCH_STATUS();
    }
#undef LAUNCH_VEC
#define LAUNCH(T)                                                                                                    \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(qk_norm_rope_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
        qk_norm_rope_kernel<T><<<n_tokens, 256, smem, stream>>>((const T*)qkv, ld, bias, q_gain, k_gain, eps,       \
                                                                positions, seq_of_token, block_table, bt_stride,     \
                                                                inv_freq, magnitude, (T*)q_out, (T*)k_pages,         \
                                                                (T*)v_pages, H, G, D, V, rotary_dim, page_size, head_unit);     \
    } while (0)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}
