// Lightning attention: linear attention with a fixed decay per head and a matrix state per request.
//
//   q = silu(W_q h), k = silu(W_k h)  [H, D];   v = silu(W_v h)  [H, V]          (the projections come in `proj`)
//   S_t = decay_h * S_(t-1) + k_t v_t^T  (S [D, V] per head, FP32, zero at a sequence's start);   o_t = S_t^T q_t
//   y = (o over all heads / sqrt(mean(o^2) + eps) * weight) * sigmoid(W_g h)
//
// Everything after the projections is FP32 whatever the tensors' type.
//
// A request's tokens of a step run in chunks of LT_C tokens.  With n tokens in a chunk, S0 the state before it and
// p[i] = decay^i (a table built by repeated multiplication, as the recurrence itself would):
//
//   A[t, j] = (q_t . k_j) p[t - j]                      for j <= t            (scores; no softmax)
//   o_t     = sum_(j <= t) A[t, j] v_j  +  p[t + 1] S0^T q_t
//   S       = p[n] S0 + sum_j p[n - 1 - j] k_j v_j^T
//
// which is the recurrence written out; only the order of the additions differs.  Chunks depend on one another only
// through S, so a step is three launches:
//
//   lightning_chunk_kv_kernel    every chunk's own sum_j p[n - 1 - j] k_j v_j^T, all chunks at once, into a buffer
//   lightning_scan_kernel        per request and head, chunk after chunk: the state BEFORE the chunk goes into the
//                                buffer's second half, the running state takes the chunk's sum; the last one is the new state
//   lightning_chunk_out_kernel   every chunk's read-out from its scores, its values and the state before it, all chunks
//                                at once
//
// and a step of single tokens is one launch (lightning_token_kernel) that reads and writes every state once.
// For FP32 projections all products are register-tiled FP32 FMA loops over shared memory.  For bfloat16 projections
// whose sizes are multiples of 16 the two chunk kernels run on tensor cores (see below), with everything the design
// keeps in 32 bits split into two bfloat16 halves.
#include "common.cuh"

#define LT_C 64          // tokens per chunk
#define LT_THREADS 256
#define LT_KV_TILE 64    // rows and columns of a chunk's sum that one block of lightning_chunk_kv_kernel owns

__device__ __forceinline__ float lt_silu(float z) { return z / (1.0f + expf(-z)); }
// The activation of a projection's entry, in the projection's own type: bfloat16 projections give the bfloat16 rounding
// of silu, in every kernel of this file alike, so that a prompt's portion and single tokens read the same q, k and v.
template <typename T> __device__ __forceinline__ float lt_act(T raw) { return ni_to_float(ni_from_float<T>(lt_silu(ni_to_float(raw)))); }
// The fast exponential and division are exact enough for a result that is rounded to 8 bits of mantissa.
template <> __device__ __forceinline__ float lt_act<__nv_bfloat16>(__nv_bfloat16 raw) {
    const float z = __bfloat162float(raw);
    return __bfloat162float(__float2bfloat16_rn(__fdividef(z, 1.0f + __expf(-z))));
}

// An FP32 entry that enters the recurrence as it is (no activation): the caller has made q, k and v itself, for
// instance rotated queries and scaled keys of a retention layer.  A type of its own, so that the FP32 FMA kernels
// below get a second instance and the ones with silu stay as they are.
struct LtPlain { float v; };
template <> __device__ __forceinline__ float ni_to_float<LtPlain>(LtPlain x) { return x.v; }
template <> __device__ __forceinline__ float lt_act<LtPlain>(LtPlain raw) { return raw.v; }

// dst[r * dst_stride + c] = f(src[r * ld + c]) * scale[r] for r < rows, c < cols (zero for rows .. rows_pad - 1 and
// c in cols .. cols_pad - 1).  16 bytes per load when every row starts on 16 bytes and cols is a multiple of the
// vector's elements.
template <typename T, bool SILU>
__device__ __forceinline__ void lt_load_tile(const T* __restrict__ src, size_t ld, int rows, int rows_pad, int cols, int cols_pad,
                                             float* __restrict__ dst, int dst_stride, const float* __restrict__ row_scale,
                                             int scale_last) {
    constexpr int VEC = 16 / sizeof(T);
    const bool wide = cols % VEC == 0 && ld % VEC == 0 && (reinterpret_cast<size_t>(src) & 15) == 0 && cols_pad % 4 == 0 &&
                      dst_stride % 4 == 0;
    if (wide) {
        const int per_row = cols_pad / VEC + (cols_pad % VEC ? 1 : 0);
        for (int i = threadIdx.x; i < rows_pad * per_row; i += LT_THREADS) {
            const int r = i / per_row, c = (i - r * per_row) * VEC;
            float v[VEC];
            if (r < rows && c < cols) {
                const uint4 raw = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + c);
                const T* e = reinterpret_cast<const T*>(&raw);
                const float sc = row_scale ? row_scale[scale_last - r] : 1.0f;
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    v[k] = (SILU ? lt_act<T>(e[k]) : ni_to_float(e[k])) * sc;
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) v[k] = 0.f;
            }
#pragma unroll
            for (int k = 0; k < VEC; k += 4)
                if (c + k < cols_pad)
                    *reinterpret_cast<float4*>(dst + r * dst_stride + c + k) = make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]);
        }
        return;
    }
    for (int i = threadIdx.x; i < rows_pad * cols_pad; i += LT_THREADS) {
        const int r = i / cols_pad, c = i - r * cols_pad;
        float v = 0.f;
        if (r < rows && c < cols) {
            const T raw = src[(size_t)r * ld + c];
            v = (SILU ? lt_act<T>(raw) : ni_to_float(raw)) * (row_scale ? row_scale[scale_last - r] : 1.0f);
        }
        dst[r * dst_stride + c] = v;
    }
}

// The first chunk of request `seq` in the buffer: the chunks of the requests before it, counted by all threads.
__device__ __forceinline__ int lt_chunk_base(const int* __restrict__ cu_q, int seq, int* scratch) {
    if (threadIdx.x == 0) *scratch = 0;
    __syncthreads();
    int mine = 0;
    for (int s = threadIdx.x; s < seq; s += blockDim.x) mine += (cu_q[s + 1] - cu_q[s] + LT_C - 1) / LT_C;
    if (mine) atomicAdd(scratch, mine);
    __syncthreads();
    return *scratch;
}

// grid (chunks of the longest request x row tiles x column tiles, H, requests); buf [chunks, H, D, V]
template <typename T>
__global__ void __launch_bounds__(LT_THREADS)
lightning_chunk_kv_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ cu_q, const float* __restrict__ decay,
                          float* __restrict__ buf, int H, int D, int V, int d_tiles, int v_tiles) {
    __shared__ __align__(16) float Ks[LT_C][LT_KV_TILE];
    __shared__ __align__(16) float Vs[LT_C][LT_KV_TILE];
    __shared__ float pw[LT_C + 1];
    __shared__ int base_s;
    const int tid = threadIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int chunk = blockIdx.x / (d_tiles * v_tiles), tile = blockIdx.x % (d_tiles * v_tiles);
    const int d0 = (tile / v_tiles) * LT_KV_TILE, v0 = (tile % v_tiles) * LT_KV_TILE;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int c0 = t0 + chunk * LT_C;
    if (c0 >= t1) return;
    const int base = lt_chunk_base(cu_q, seq, &base_s);
    const int n = min(LT_C, t1 - c0);
    if (tid == 0) {
        const float dec = decay[head];
        float p = 1.0f;
        for (int i = 0; i <= LT_C; ++i) { pw[i] = p; p *= dec; }
    }
    __syncthreads();
    const T* xk = proj + (size_t)(H + head) * D + d0;
    const T* xv = proj + (size_t)2 * H * D + (size_t)head * V + v0;
    lt_load_tile<T, true>(xk + (size_t)c0 * ld, ld, n, n, min(LT_KV_TILE, D - d0), LT_KV_TILE, &Ks[0][0], LT_KV_TILE, nullptr, 0);
    lt_load_tile<T, true>(xv + (size_t)c0 * ld, ld, n, n, min(LT_KV_TILE, V - v0), LT_KV_TILE, &Vs[0][0], LT_KV_TILE, pw, n - 1);   // decayed to the chunk's end
    __syncthreads();
    const int vg = (tid % 16) * 4, dg = (tid / 16) * 4;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
    for (int j = 0; j < n; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(&Ks[j][dg]);
        const float4 v4 = *reinterpret_cast<const float4*>(&Vs[j][vg]);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(kk[a], vv[b], acc[a][b]);
    }
    float* out = buf + ((size_t)(base + chunk) * H + head) * D * V;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (d0 + dg + a < D && v0 + vg + b < V) out[(size_t)(d0 + dg + a) * V + v0 + vg + b] = acc[a][b];
}

// grid (ceil(D V / threads), H, requests).  sums [chunks, H, D, V] in, before [chunks, H, D, V] out: FP32, or with
// `split` two bfloat16 planes [2, D, V] per chunk and head (hi, then lo = the rounding of the remainder) in the same bytes.
__global__ void lightning_scan_kernel(float* __restrict__ state, long long state_stride, const int* __restrict__ cu_q,
                                      const int* __restrict__ slots, const float* __restrict__ decay,
                                      const float* __restrict__ sums, float* __restrict__ before, int split, int H, int D, int V) {
    __shared__ int base_s;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int len = cu_q[seq + 1] - cu_q[seq];
    if (len <= 0) return;
    const int base = lt_chunk_base(cu_q, seq, &base_s);
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= D * V) return;
    const float dec = decay[head];
    float p_full = 1.0f;
    for (int i = 0; i < LT_C; ++i) p_full *= dec;
    float* S = state + (size_t)slots[seq] * state_stride + (size_t)head * D * V + e;
    float s = *S;
    const size_t stride = (size_t)H * D * V, first = ((size_t)base * H + head) * D * V;
    const float* b = sums + first + e;
    float* o32 = before + first + e;
    __nv_bfloat16* o16 = reinterpret_cast<__nv_bfloat16*>(before + first) + e;
    const int chunks = (len + LT_C - 1) / LT_C;
    for (int c = 0; c < chunks; c += 8) {
        float own[8];                             // loaded together: the chain below waits for memory once per group
#pragma unroll
        for (int i = 0; i < 8; ++i) own[i] = c + i < chunks ? b[(size_t)(c + i) * stride] : 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (c + i >= chunks) break;
            const int n = min(LT_C, len - (c + i) * LT_C);
            float pn = p_full;
            if (n < LT_C) {
                pn = 1.0f;
                for (int k = 0; k < n; ++k) pn *= dec;
            }
            if (split) {                           // what the chunk's read-out starts from
                const __nv_bfloat16 hi = __float2bfloat16_rn(s);
                o16[(size_t)(c + i) * stride * 2] = hi;
                o16[(size_t)(c + i) * stride * 2 + (size_t)D * V] = __float2bfloat16_rn(s - __bfloat162float(hi));
            } else {
                o32[(size_t)(c + i) * stride] = s;
            }
            s = fmaf(pn, s, own[i]);
        }
    }
    *S = s;
}

// grid (chunks of the longest request x column tiles of VT, H, requests); buf holds the state before every chunk
template <typename T, int VT>
__global__ void __launch_bounds__(LT_THREADS)
lightning_chunk_out_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ cu_q, const float* __restrict__ decay,
                           const float* __restrict__ buf, float* __restrict__ out, int H, int D, int V, int v_tiles) {
    extern __shared__ __align__(16) float sm[];
    __shared__ int base_s;
    constexpr int TT = LT_C * VT / (LT_THREADS * 4);        // tokens per thread of the read-out (4 columns each)
    constexpr int AS = LT_C + 4;
    const int DP = (D + 3) & ~3;             // rows padded to whole float4s (zeros)
    const int QS = DP + 4;                   // row stride of Qs / Ks: neighbouring rows start 4 banks apart
    float* Ss = sm;                          // [DP][VT]
    float* Qs = Ss + DP * VT;                // [LT_C][QS]
    float* Ks = Qs + LT_C * QS;              // [LT_C][QS]
    float* Vs = Ks + LT_C * QS;              // [LT_C][VT]
    float* As = Vs + LT_C * VT;              // [LT_C][AS]
    float* pw = As + LT_C * AS;              // [LT_C + 1]

    const int tid = threadIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int chunk = blockIdx.x / v_tiles, v0 = (blockIdx.x % v_tiles) * VT;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int c0 = t0 + chunk * LT_C;
    if (c0 >= t1) return;
    const int base = lt_chunk_base(cu_q, seq, &base_s);
    const int n = min(LT_C, t1 - c0), n4 = (n + 3) & ~3;
    const int vt = min(VT, V - v0);
    if (tid == 0) {
        const float dec = decay[head];
        float p = 1.0f;
        for (int i = 0; i <= LT_C; ++i) { pw[i] = p; p *= dec; }
    }
    const float* S0 = buf + ((size_t)(base + chunk) * H + head) * D * V + v0;
    lt_load_tile<float, false>(S0, V, D, DP, vt, VT, Ss, VT, nullptr, 0);
    lt_load_tile<T, true>(proj + (size_t)c0 * ld + (size_t)head * D, ld, n, n4, D, DP, Qs, QS, nullptr, 0);
    lt_load_tile<T, true>(proj + (size_t)c0 * ld + (size_t)(H + head) * D, ld, n, n4, D, DP, Ks, QS, nullptr, 0);
    lt_load_tile<T, true>(proj + (size_t)c0 * ld + (size_t)2 * H * D + (size_t)head * V + v0, ld, n, n4, vt, VT, Vs, VT, nullptr, 0);
    __syncthreads();
    // ---- scores: A[t, j] = (q_t . k_j) p[t - j], zero above the diagonal; a thread owns one 4 x 4 tile on or below it
    if (tid < (LT_C / 4) * (LT_C / 4 + 1) / 2) {
        int ti = 0, ji = tid;
        while (ji > ti) { ji -= ti + 1; ++ti; }
        if (ti * 4 < n4) {
            float acc[4][4];
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
            const float* qp = Qs + ti * 4 * QS;
            const float* kp = Ks + ji * 4 * QS;
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
                    const int t = ti * 4 + a, j = ji * 4 + b;
                    As[t * AS + j] = j <= t ? acc[a][b] * pw[t - j] : 0.f;
                }
        }
    }
    __syncthreads();
    // ---- read-out: o_t = sum_(j <= t) A[t, j] v_j + p[t + 1] S0^T q_t; a thread owns TT tokens x 4 value columns
    const int vg = (tid % (VT / 4)) * 4, tg = (tid / (VT / 4)) * TT;
    if (tg >= n4) return;
    float intra[TT][4], inter[TT][4];
#pragma unroll
    for (int a = 0; a < TT; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) intra[a][b] = inter[a][b] = 0.f;
    const int j_end = (tg + TT + 3) & ~3;                     // scores beyond the diagonal are zero
    for (int j = 0; j < j_end; j += 4) {
        float4 av[TT], wv[4];
#pragma unroll
        for (int a = 0; a < TT; ++a) av[a] = *reinterpret_cast<const float4*>(As + (tg + a) * AS + j);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) wv[jj] = *reinterpret_cast<const float4*>(Vs + (j + jj) * VT + vg);
#pragma unroll
        for (int a = 0; a < TT; ++a) {
            const float aa[4] = {av[a].x, av[a].y, av[a].z, av[a].w};
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                intra[a][0] = fmaf(aa[jj], wv[jj].x, intra[a][0]);
                intra[a][1] = fmaf(aa[jj], wv[jj].y, intra[a][1]);
                intra[a][2] = fmaf(aa[jj], wv[jj].z, intra[a][2]);
                intra[a][3] = fmaf(aa[jj], wv[jj].w, intra[a][3]);
            }
        }
    }
    for (int d = 0; d < DP; d += 4) {
        float4 qv[TT], sv[4];
#pragma unroll
        for (int a = 0; a < TT; ++a) qv[a] = *reinterpret_cast<const float4*>(Qs + (tg + a) * QS + d);
#pragma unroll
        for (int dd = 0; dd < 4; ++dd) sv[dd] = *reinterpret_cast<const float4*>(Ss + (d + dd) * VT + vg);
#pragma unroll
        for (int a = 0; a < TT; ++a) {
            const float qq[4] = {qv[a].x, qv[a].y, qv[a].z, qv[a].w};
#pragma unroll
            for (int dd = 0; dd < 4; ++dd) {
                inter[a][0] = fmaf(qq[dd], sv[dd].x, inter[a][0]);
                inter[a][1] = fmaf(qq[dd], sv[dd].y, inter[a][1]);
                inter[a][2] = fmaf(qq[dd], sv[dd].z, inter[a][2]);
                inter[a][3] = fmaf(qq[dd], sv[dd].w, inter[a][3]);
            }
        }
    }
#pragma unroll
    for (int a = 0; a < TT; ++a) {
        const int t = tg + a;
        if (t >= n) continue;
        float* o = out + (size_t)(c0 + t) * H * V + (size_t)head * V + v0 + vg;
#pragma unroll
        for (int b = 0; b < 4; ++b)
            if (vg + b < vt) o[b] = fmaf(pw[t + 1], inter[a][b], intra[a][b]);
    }
}

// ---- bfloat16 projections: the same two chunk kernels on tensor cores ------------------------------------------------
// mma.sync m16n8k16 (bfloat16 operands, FP32 accumulation).  q, k and v enter as the bfloat16 roundings of their
// activations.  Whatever the design keeps in 32 bits and a product has to read again - the decayed scores, the state
// before the chunk, the decayed keys of a chunk's sum - is split into two bfloat16 numbers x = hi + lo (lo the rounding
// of x - hi), and the product runs once with each: 16 bits of mantissa instead of 8, in FP32 accumulators.
__device__ __forceinline__ void lt_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Four 8 x 8 blocks of 16-bit numbers, each transposed on the way: lane l gives the address of row l % 8 of block l / 8.
__device__ __forceinline__ void lt_ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lt_split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ void lt_cp_async16(void* smem, const void* gmem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem));
}
__device__ __forceinline__ void lt_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
// Waits until at most N of the thread's committed groups are still under way.
template <int N> __device__ __forceinline__ void lt_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
// Rows [0, rows) x columns [0, cols) of src copied as they are (asynchronously, 16 bytes a piece) into dst, zeros up to
// rows_pad x cols_pad; lt_activate_own then turns the pieces that the same thread copied into their activations, in place
// (times scale[scale_last - r], the remainder of the rounding into dst_lo if given).
// Calls piece(r, c) for every 8-number piece (row r, first column c) of rows x cols_pad, thread by thread; the same thread
// gets the same pieces in every call with the same sizes.  When a row's pieces divide the block, a thread keeps its
// column and steps down the rows (no division per piece).
template <int THREADS, typename F>
__device__ __forceinline__ void lt_for_pieces(int rows, int cols_pad, F piece) {
    const int per_row = cols_pad / 8;
    if (THREADS % per_row == 0) {
        const int c = (threadIdx.x % per_row) * 8, dr = THREADS / per_row;
#pragma unroll 4
        for (int r = threadIdx.x / per_row; r < rows; r += dr) piece(r, c);
    } else {
        for (int i = threadIdx.x; i < rows * per_row; i += THREADS) piece(i / per_row, (i % per_row) * 8);
    }
}
template <int THREADS>
__device__ __forceinline__ void lt_copy_raw(const __nv_bfloat16* __restrict__ src, size_t ld, int rows, int rows_pad, int cols,
                                            int cols_pad, __nv_bfloat16* __restrict__ dst, int dst_stride) {
    lt_for_pieces<THREADS>(rows_pad, cols_pad, [&](int r, int c) {
        if (r < rows && c < cols) lt_cp_async16(dst + r * dst_stride + c, src + (size_t)r * ld + c);
        else *reinterpret_cast<uint4*>(dst + r * dst_stride + c) = make_uint4(0u, 0u, 0u, 0u);
    });
}
template <int THREADS>
__device__ __forceinline__ void lt_activate_own(int rows, int cols, int cols_pad, __nv_bfloat16* __restrict__ dst_hi,
                                                __nv_bfloat16* __restrict__ dst_lo, int dst_stride,
                                                const float* __restrict__ row_scale, int scale_last) {
    lt_for_pieces<THREADS>(rows, cols_pad, [&](int r, int c) {
        if (c >= cols) return;
        uint4 raw = *reinterpret_cast<const uint4*>(dst_hi + r * dst_stride + c), lo;
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&raw);
        const float sc = row_scale ? row_scale[scale_last - r] : 1.0f;
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = lt_act<__nv_bfloat16>(e[k]) * sc;
        lt_split2(v[0], v[1], raw.x, lo.x);
        lt_split2(v[2], v[3], raw.y, lo.y);
        lt_split2(v[4], v[5], raw.z, lo.z);
        lt_split2(v[6], v[7], raw.w, lo.w);
        *reinterpret_cast<uint4*>(dst_hi + r * dst_stride + c) = raw;
        if (dst_lo) *reinterpret_cast<uint4*>(dst_lo + r * dst_stride + c) = lo;
    });
}

// grid (chunks of the longest request, H, requests); a block owns its chunk's whole sum: a warp 16 rows of it at a time,
// 64 columns at a time.  D and V multiples of 16.
__global__ void __launch_bounds__(LT_THREADS)
lightning_chunk_kv_tc_kernel(const __nv_bfloat16* __restrict__ proj, int ld, const int* __restrict__ cu_q,
                             const float* __restrict__ decay, float* __restrict__ buf, int H, int D, int V) {
    extern __shared__ __align__(16) unsigned char lt_raw[];
    __shared__ float pw[LT_C + 1];
    __shared__ int base_s;
    const int KS = D + 8, VS = V + 8;
    __nv_bfloat16* Khi = reinterpret_cast<__nv_bfloat16*>(lt_raw);      // [LT_C][KS] keys decayed to the chunk's end
    __nv_bfloat16* Klo = Khi + LT_C * KS;
    __nv_bfloat16* Vs = Klo + LT_C * KS;                                // [LT_C][VS]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunk = blockIdx.x, head = blockIdx.y, seq = blockIdx.z;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int c0 = t0 + chunk * LT_C;
    if (c0 >= t1) return;
    const int base = lt_chunk_base(cu_q, seq, &base_s);
    const int n = min(LT_C, t1 - c0);
    if (tid == 0) {
        const float dec = decay[head];
        float p = 1.0f;
        for (int i = 0; i <= LT_C; ++i) { pw[i] = p; p *= dec; }
    }
    __syncthreads();
    const __nv_bfloat16* row0 = proj + (size_t)c0 * ld;
    lt_copy_raw<LT_THREADS>(row0 + (size_t)(H + head) * D, ld, n, LT_C, D, D, Khi, KS);
    lt_cp_async_commit();
    lt_copy_raw<LT_THREADS>(row0 + (size_t)2 * H * D + (size_t)head * V, ld, n, LT_C, V, V, Vs, VS);
    lt_cp_async_commit();
    for (int i = tid; i < (LT_C - n) * (D / 8); i += LT_THREADS)          // the rows beyond the chunk's tokens
        *reinterpret_cast<uint4*>(Klo + (n + i / (D / 8)) * KS + (i % (D / 8)) * 8) = make_uint4(0u, 0u, 0u, 0u);
    lt_cp_async_wait<1>();                                 // the keys are here; the values are still under way
    lt_activate_own<LT_THREADS>(n, D, D, Khi, Klo, KS, pw, n - 1);
    lt_cp_async_wait<0>();
    lt_activate_own<LT_THREADS>(n, V, V, Vs, nullptr, VS, nullptr, 0);
    __syncthreads();
    const int g = lane >> 2, tq = lane & 3, blk = lane >> 3, rr = lane & 7;
    const int k_steps = (n + 15) / 16;
    float* out = buf + ((size_t)(base + chunk) * H + head) * D * V;
    for (int mt = warp; mt < D / 16; mt += LT_THREADS / 32) {
        const int d0 = mt * 16;
        for (int vb = 0; vb < V; vb += 64) {
            const int pairs = min(4, (V - vb) / 16);
            float acc[8][4];
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
            for (int kt = 0; kt < k_steps; ++kt) {
                const int j0 = kt * 16;
                uint32_t ahi[4], alo[4];
                const int a_off = (j0 + (blk >> 1) * 8 + rr) * KS + d0 + (blk & 1) * 8;
                lt_ldsm_x4_trans(ahi, Khi + a_off);
                lt_ldsm_x4_trans(alo, Klo + a_off);
                const __nv_bfloat16* vp = Vs + (j0 + (blk & 1) * 8 + rr) * VS + vb + (blk >> 1) * 8;
                if (pairs == 4) {                               // a whole block of 64 columns: no checks between the loads
                    uint32_t b[4][4];
#pragma unroll
                    for (int np = 0; np < 4; ++np) lt_ldsm_x4_trans(b[np], vp + np * 16);
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        lt_mma(acc[2 * np], ahi, b[np][0], b[np][1]);
                        lt_mma(acc[2 * np + 1], ahi, b[np][2], b[np][3]);
                    }
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        lt_mma(acc[2 * np], alo, b[np][0], b[np][1]);
                        lt_mma(acc[2 * np + 1], alo, b[np][2], b[np][3]);
                    }
                } else {
#pragma unroll
                    for (int np = 0; np < 4; ++np) {
                        if (np < pairs) {
                            uint32_t b[4];
                            lt_ldsm_x4_trans(b, vp + np * 16);
                            lt_mma(acc[2 * np], ahi, b[0], b[1]);
                            lt_mma(acc[2 * np], alo, b[0], b[1]);
                            lt_mma(acc[2 * np + 1], ahi, b[2], b[3]);
                            lt_mma(acc[2 * np + 1], alo, b[2], b[3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (nt < 2 * pairs) {
                    const int col = vb + nt * 8 + 2 * tq;
                    *reinterpret_cast<float2*>(out + (size_t)(d0 + g) * V + col) = make_float2(acc[nt][0], acc[nt][1]);
                    *reinterpret_cast<float2*>(out + (size_t)(d0 + g + 8) * V + col) = make_float2(acc[nt][2], acc[nt][3]);
                }
            }
        }
    }
}

// The three phases of one warp of lightning_chunk_out_tc_kernel: tokens MW * 16 .. MW * 16 + 15 of the chunk, columns
// vh .. vh + 16 pairs - 1 of the block's tile (FULL: all 64, no column checks inside the loops).  One instance of the
// loops serves all warps: tiles beyond a warp's diagonal are skipped by a branch that the whole warp takes alike.
// Scores of the warp's 16 tokens with the keys up to their diagonal block, decayed and masked.
__device__ __forceinline__ void lt_out_scores(const __nv_bfloat16* __restrict__ Qs, const __nv_bfloat16* __restrict__ Ks,
                                              const float* __restrict__ pw, int QS, int D, int MW, float (&sc)[8][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int r0 = MW * 16;
    for (int kk = 0; kk < D; kk += 16) {
        uint32_t a[4];
        const __nv_bfloat16* qp = Qs + (r0 + g) * QS + kk + 2 * tq;
        a[0] = *reinterpret_cast<const uint32_t*>(qp);
        a[1] = *reinterpret_cast<const uint32_t*>(qp + 8 * QS);
        a[2] = *reinterpret_cast<const uint32_t*>(qp + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(qp + 8 * QS + 8);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            if (nt < 2 * MW + 2) {
                const __nv_bfloat16* kp = Ks + (nt * 8 + g) * QS + kk + 2 * tq;
                lt_mma(sc[nt], a, *reinterpret_cast<const uint32_t*>(kp), *reinterpret_cast<const uint32_t*>(kp + 8));
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = r0 + g + (i >> 1) * 8, j = nt * 8 + 2 * tq + (i & 1);
            sc[nt][i] = j <= t ? sc[nt][i] * pw[t - j] : 0.f;
        }
}
// What the state before the chunk gives: p[t + 1] S0^T q_t.
template <bool FULL>
__device__ __forceinline__ void lt_out_inter(const __nv_bfloat16* __restrict__ Qs, const __nv_bfloat16* __restrict__ Shi,
                                             const __nv_bfloat16* __restrict__ Slo, const float* __restrict__ pw, int QS, int VS,
                                             int D, int r0, int vh, int pairs, float (&acc)[8][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3, blk = lane >> 3, rr = lane & 7;
    for (int kk = 0; kk < D; kk += 16) {
        uint32_t a[4];
        const __nv_bfloat16* qp = Qs + (r0 + g) * QS + kk + 2 * tq;
        a[0] = *reinterpret_cast<const uint32_t*>(qp);
        a[1] = *reinterpret_cast<const uint32_t*>(qp + 8 * QS);
        a[2] = *reinterpret_cast<const uint32_t*>(qp + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(qp + 8 * QS + 8);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            if (FULL || np < pairs) {
                const int off = (kk + (blk & 1) * 8 + rr) * VS + vh + np * 16 + (blk >> 1) * 8;
                uint32_t b[4];
                lt_ldsm_x4_trans(b, Shi + off);
                lt_mma(acc[2 * np], a, b[0], b[1]);
                lt_mma(acc[2 * np + 1], a, b[2], b[3]);
                lt_ldsm_x4_trans(b, Slo + off);
                lt_mma(acc[2 * np], a, b[0], b[1]);
                lt_mma(acc[2 * np + 1], a, b[2], b[3]);
            }
        }
    }
    const float p_lo = pw[min(r0 + g + 1, LT_C)], p_hi = pw[min(r0 + g + 9, LT_C)];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        acc[nt][0] *= p_lo;
        acc[nt][1] *= p_lo;
        acc[nt][2] *= p_hi;
        acc[nt][3] *= p_hi;
    }
}
// What the chunk's own tokens give, sum_(j <= t) A[t, j] v_j, added; then the warp's rows of the output.
template <bool FULL>
__device__ __forceinline__ void lt_out_intra(const float (&sc)[8][4], const __nv_bfloat16* __restrict__ Vs, int VS, int vh, int pairs,
                                             int n, int MW, float (&acc)[8][4], float* __restrict__ out, size_t out_stride) {
    const int lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3, blk = lane >> 3, rr = lane & 7;
    const int r0 = MW * 16;
#pragma unroll
    for (int kt = 0; kt < 4; ++kt) {
        if (kt <= MW) {
            uint32_t ahi[4], alo[4];
            lt_split2(sc[2 * kt][0], sc[2 * kt][1], ahi[0], alo[0]);
            lt_split2(sc[2 * kt][2], sc[2 * kt][3], ahi[1], alo[1]);
            lt_split2(sc[2 * kt + 1][0], sc[2 * kt + 1][1], ahi[2], alo[2]);
            lt_split2(sc[2 * kt + 1][2], sc[2 * kt + 1][3], ahi[3], alo[3]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                if (FULL || np < pairs) {
                    uint32_t b[4];
                    lt_ldsm_x4_trans(b, Vs + (kt * 16 + (blk & 1) * 8 + rr) * VS + vh + np * 16 + (blk >> 1) * 8);
                    lt_mma(acc[2 * np], ahi, b[0], b[1]);
                    lt_mma(acc[2 * np], alo, b[0], b[1]);
                    lt_mma(acc[2 * np + 1], ahi, b[2], b[3]);
                    lt_mma(acc[2 * np + 1], alo, b[2], b[3]);
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        if (FULL || nt < 2 * pairs) {
            const int col = vh + nt * 8 + 2 * tq;
            const int ta = r0 + g, tb = r0 + g + 8;
            if (ta < n) *reinterpret_cast<float2*>(out + (size_t)ta * out_stride + col) = make_float2(acc[nt][0], acc[nt][1]);
            if (tb < n) *reinterpret_cast<float2*>(out + (size_t)tb * out_stride + col) = make_float2(acc[nt][2], acc[nt][3]);
        }
    }
}

// grid (chunks of the longest request x column tiles of VT, H, requests); VT 64 or 128; VT / 64 groups of four warps,
// a group owns 64 columns, a warp of it 16 tokens of the chunk (the groups compute the same scores).  The values are
// copied after the scores, into the keys' place when they fit there (D >= VT: `v_in_k`), while the warps multiply with
// the state before the chunk; that leaves room for two blocks on an SM at 128 x 128 heads.
template <int VT>
__global__ void __launch_bounds__(VT * 2, VT == 128 ? 2 : 3)
lightning_chunk_out_tc_kernel(const __nv_bfloat16* __restrict__ proj, int ld, const int* __restrict__ cu_q,
                              const float* __restrict__ decay, const float* __restrict__ buf, float* __restrict__ out,
                              int H, int D, int V, int v_tiles, int v_in_k) {
    extern __shared__ __align__(16) unsigned char lt_raw[];
    __shared__ float pw[LT_C + 1];
    __shared__ int base_s;
    constexpr int VS = VT + 8, LT_OUT_TC_THREADS = VT * 2;
    const int QS = D + 8;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(lt_raw);       // [LT_C][QS]
    __nv_bfloat16* Ks = Qs + LT_C * QS;                                 // [LT_C][QS]
    __nv_bfloat16* Shi = Ks + LT_C * QS;                                // [D][VS] the state before the chunk
    __nv_bfloat16* Slo = Shi + D * VS;
    __nv_bfloat16* Vs = v_in_k ? Ks : Slo + D * VS;                     // [LT_C][VS]
    const int tid = threadIdx.x, warp = tid >> 5;
    const int head = blockIdx.y, seq = blockIdx.z;
    const int chunk = blockIdx.x / v_tiles, v0 = (blockIdx.x % v_tiles) * VT;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    const int c0 = t0 + chunk * LT_C;
    if (c0 >= t1) return;
    const int base = lt_chunk_base(cu_q, seq, &base_s);
    const int n = min(LT_C, t1 - c0);
    const int vt = min(VT, V - v0);
    if (tid == 0) {
        const float dec = decay[head];
        float p = 1.0f;
        for (int i = 0; i <= LT_C; ++i) { pw[i] = p; p *= dec; }
    }
    const __nv_bfloat16* S0 = reinterpret_cast<const __nv_bfloat16*>(buf + ((size_t)(base + chunk) * H + head) * D * V) + v0;
    const __nv_bfloat16* row0 = proj + (size_t)c0 * ld;
    lt_copy_raw<LT_OUT_TC_THREADS>(row0 + (size_t)head * D, ld, n, LT_C, D, D, Qs, QS);
    lt_copy_raw<LT_OUT_TC_THREADS>(row0 + (size_t)(H + head) * D, ld, n, LT_C, D, D, Ks, QS);
    lt_cp_async_commit();
    lt_copy_raw<LT_OUT_TC_THREADS>(S0, V, D, D, vt, VT, Shi, VS);                  // the two planes of the state before
    lt_copy_raw<LT_OUT_TC_THREADS>(S0 + (size_t)D * V, V, D, D, vt, VT, Slo, VS);
    lt_cp_async_commit();
    lt_cp_async_wait<1>();                                 // q and k are here; the state's planes are still under way
    lt_activate_own<LT_OUT_TC_THREADS>(n, D, D, Qs, nullptr, QS, nullptr, 0);
    lt_activate_own<LT_OUT_TC_THREADS>(n, D, D, Ks, nullptr, QS, nullptr, 0);
    __syncthreads();
    const int mw = warp & 3, vh = (warp >> 2) * 64;       // the warp's tokens and its columns of the tile
    const bool active = mw * 16 < n && vh < vt;           // the others only copy and wait with the block
    const int pairs = min(4, max(0, vt - vh) / 16);
    float sc[8][4], acc[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) sc[a][b] = acc[a][b] = 0.f;
    if (active) lt_out_scores(Qs, Ks, pw, QS, D, mw, sc);
    lt_cp_async_wait<0>();
    __syncthreads();                                      // the state's planes are here; nobody reads the keys any more
    lt_copy_raw<LT_OUT_TC_THREADS>(row0 + (size_t)2 * H * D + (size_t)head * V + v0, ld, n, LT_C, vt, VT, Vs, VS);
    lt_cp_async_commit();
    if (active) {
        if (pairs == 4) lt_out_inter<true>(Qs, Shi, Slo, pw, QS, VS, D, mw * 16, vh, pairs, acc);
        else lt_out_inter<false>(Qs, Shi, Slo, pw, QS, VS, D, mw * 16, vh, pairs, acc);
    }
    lt_cp_async_wait<0>();
    lt_activate_own<LT_OUT_TC_THREADS>(n, vt, VT, Vs, nullptr, VS, nullptr, 0);
    __syncthreads();
    if (!active) return;
    float* o = out + (size_t)c0 * H * V + (size_t)head * V + v0;
    if (pairs == 4) lt_out_intra<true>(sc, Vs, VS, vh, pairs, n, mw, acc, o, (size_t)H * V);
    else lt_out_intra<false>(sc, Vs, VS, vh, pairs, n, mw, acc, o, (size_t)H * V);
}

// A step of single tokens: S <- decay S + k v^T, o = S^T q; every state is read and written once.
// grid (column tiles of 128, H, requests); a warp owns every 8th row, a lane 4 neighbouring columns.
// ROT (retention): nothing is activated; instead the first rotary_dim dimensions of q and k are rotated by the token's
// position (dimension i paired with i + rotary_dim / 2, angle float(position) * inv_freq[i]) and k is multiplied by
// k_scale, all in FP32 from the projection's entries - the single-token form of linear_attention_prepare_kernel.
template <typename T, bool ROT>
__global__ void __launch_bounds__(LT_THREADS)
lightning_token_kernel(const T* __restrict__ proj, int ld, float* __restrict__ state, long long state_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ slots, const float* __restrict__ decay,
                       float* __restrict__ out, int H, int D, int V, const int* __restrict__ positions,
                       const float* __restrict__ inv_freq, int rotary_dim, float k_scale) {
    extern __shared__ __align__(16) float sm[];
    float* qs = sm;                          // [D]
    float* ks = qs + D;                      // [D]
    float* part = ks + D;                    // [8 warps][128 columns]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int v0 = blockIdx.x * 128, head = blockIdx.y, seq = blockIdx.z;
    const int t = cu_q[seq];
    if (cu_q[seq + 1] <= t) return;
    const T* row = proj + (size_t)t * ld;
    if (ROT) {
        const float pos = (float)positions[t];
        const int half = rotary_dim >> 1;
        const T* qrow = row + (size_t)head * D;
        const T* krow = row + (size_t)(H + head) * D;
        for (int d = tid; d < D; d += LT_THREADS) {
            float qv = ni_to_float(qrow[d]), kv = ni_to_float(krow[d]);
            if (d < rotary_dim) {
                const bool first = d < half;
                const int other = first ? d + half : d - half;
                float sn, cs;
                sincosf(pos * inv_freq[first ? d : d - half], &sn, &cs);
                const float qo = ni_to_float(qrow[other]), ko = ni_to_float(krow[other]);
                qv = first ? qv * cs - qo * sn : qv * cs + qo * sn;
                kv = first ? kv * cs - ko * sn : kv * cs + ko * sn;
            }
            qs[d] = qv;
            ks[d] = kv * k_scale;
        }
    } else {
        for (int d = tid; d < D; d += LT_THREADS) {
            qs[d] = lt_act<T>(row[(size_t)head * D + d]);
            ks[d] = lt_act<T>(row[(size_t)(H + head) * D + d]);
        }
    }
    const int vc = v0 + lane * 4;
    float vv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const T raw = vc + b < V ? row[(size_t)2 * H * D + (size_t)head * V + vc + b] : row[0];
        vv[b] = vc + b < V ? (ROT ? ni_to_float(raw) : lt_act<T>(raw)) : 0.f;
    }
    __syncthreads();
    const float dec = decay[head];
    float* S = state + (size_t)slots[seq] * state_stride + (size_t)head * D * V;
    const bool wide = (V % 4 == 0) && ((reinterpret_cast<size_t>(S) & 15) == 0) && vc + 3 < V;
    constexpr int WARPS = LT_THREADS / 32;
    if (wide) {
        for (int d = warp; d < D; d += 4 * WARPS) {          // four rows' loads are under way before the first store
            float4 s4[4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
                if (d + r * WARPS < D) s4[r] = *reinterpret_cast<const float4*>(S + (size_t)(d + r * WARPS) * V + vc);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int dr = d + r * WARPS;
                if (dr >= D) break;
                const float k = ks[dr], q = qs[dr];
                s4[r].x = fmaf(dec, s4[r].x, k * vv[0]);
                s4[r].y = fmaf(dec, s4[r].y, k * vv[1]);
                s4[r].z = fmaf(dec, s4[r].z, k * vv[2]);
                s4[r].w = fmaf(dec, s4[r].w, k * vv[3]);
                *reinterpret_cast<float4*>(S + (size_t)dr * V + vc) = s4[r];
                acc[0] = fmaf(s4[r].x, q, acc[0]);
                acc[1] = fmaf(s4[r].y, q, acc[1]);
                acc[2] = fmaf(s4[r].z, q, acc[2]);
                acc[3] = fmaf(s4[r].w, q, acc[3]);
            }
        }
    } else {
        for (int d = warp; d < D; d += WARPS) {
            float* sp = S + (size_t)d * V + vc;
            const float k = ks[d], q = qs[d];
#pragma unroll
            for (int b = 0; b < 4; ++b)
                if (vc + b < V) {
                    const float s1 = fmaf(dec, sp[b], k * vv[b]);
                    sp[b] = s1;
                    acc[b] = fmaf(s1, q, acc[b]);
                }
        }
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) part[warp * 128 + lane * 4 + b] = acc[b];
    __syncthreads();
    if (tid < 128 && v0 + tid < V) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < LT_THREADS / 32; ++w) o += part[w * 128 + tid];
        out[(size_t)t * H * V + (size_t)head * V + v0 + tid] = o;
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

// The same with 8 numbers per thread and pass (16-byte loads of the gate, two of o; N a multiple of 8, rows on 16 bytes):
// a thread's first 8 numbers, their gates and weights stay in registers across the reduction.
__global__ void lightning_gated_norm_vec_kernel(const float* __restrict__ o, const __nv_bfloat16* __restrict__ proj, int ld, int col0,
                                                const float* __restrict__ weight, float eps, __nv_bfloat16* __restrict__ y, int N) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, first = threadIdx.x * 8, step = blockDim.x * 8;
    const float* row = o + (size_t)t * N;
    const __nv_bfloat16* g = proj + (size_t)t * ld + col0;
    float x[8], w[8];
    uint4 graw = make_uint4(0u, 0u, 0u, 0u);
    float ss = 0.f;
    if (first < N) {
        const float4 a = *reinterpret_cast<const float4*>(row + first), b = *reinterpret_cast<const float4*>(row + first + 4);
        const float4 wa = *reinterpret_cast<const float4*>(weight + first), wb = *reinterpret_cast<const float4*>(weight + first + 4);
        graw = *reinterpret_cast<const uint4*>(g + first);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        w[0] = wa.x; w[1] = wa.y; w[2] = wa.z; w[3] = wa.w; w[4] = wb.x; w[5] = wb.y; w[6] = wb.z; w[7] = wb.w;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(x[k], x[k], ss);
    }
    for (int i = first + step; i < N; i += step) {
        const float4 a = *reinterpret_cast<const float4*>(row + i), b = *reinterpret_cast<const float4*>(row + i + 4);
        ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
    }
    ss = ni_block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = first; i < N; i += step) {
        if (i != first) {
            const float4 a = *reinterpret_cast<const float4*>(row + i), b = *reinterpret_cast<const float4*>(row + i + 4);
            const float4 wa = *reinterpret_cast<const float4*>(weight + i), wb = *reinterpret_cast<const float4*>(weight + i + 4);
            graw = *reinterpret_cast<const uint4*>(g + i);
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            w[0] = wa.x; w[1] = wa.y; w[2] = wa.z; w[3] = wa.w; w[4] = wb.x; w[5] = wb.y; w[6] = wb.z; w[7] = wb.w;
        }
        const __nv_bfloat16* ge = reinterpret_cast<const __nv_bfloat16*>(&graw);
        uint4 outv;
        __nv_bfloat16* oe = reinterpret_cast<__nv_bfloat16*>(&outv);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gate = 1.0f / (1.0f + expf(-__bfloat162float(ge[k])));
            oe[k] = __float2bfloat16_rn(x[k] * inv * w[k] * gate);
        }
        *reinterpret_cast<uint4*>(y + (size_t)t * N + i) = outv;
    }
}

static size_t lt_out_smem_bytes(int D, int VT) {
    const int DP = (D + 3) & ~3;
    return ((size_t)DP * VT + 2 * (size_t)LT_C * (DP + 4) + (size_t)LT_C * VT + (size_t)LT_C * (LT_C + 4) + LT_C + 1) * sizeof(float);
}

// The most chunks that requests of n_tokens tokens in all can have.
static long long lt_chunks(int n_tokens, int n_seqs) {
    const long long whole = (long long)n_tokens / LT_C + n_seqs;
    return whole < n_tokens ? whole : n_tokens;
}
// The buffer of a step in units of H D V floats: every chunk's own sum, and the state before every chunk.
NI_EXPORT int ni_lightning_max_chunks(int n_tokens, int n_seqs) { return (int)(2 * lt_chunks(n_tokens, n_seqs)); }

// proj [T, ld] with columns q (H D) | k (H D) | v (H V) | ...; state FP32 [slots, state_stride] holding S [H, D, V] of
// every request; decay FP32 [H]; out FP32 [T, H V].  The state advances by the step's tokens.  max_q_len: the most
// tokens that one request brings (1: a step of single tokens, which needs no buffer); buf FP32 with room for
// buf_chunks x H D V, at least ni_lightning_max_chunks(n_tokens, n_seqs) of them.  activation 1: q, k, v = silu of
// proj's entries; 0: proj (FP32 only) holds q, k and v themselves.
NI_EXPORT int ni_lightning_recurrence(const void* proj, int dtype, int ld, float* state, long long state_stride,
                                      const int* cu_q, const int* slots, const float* decay, float* out, int n_tokens,
                                      int n_seqs, int max_q_len, float* buf, long long buf_chunks, int H, int D, int V,
                                      int activation, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return NI_OK;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + H * V || state_stride < (long long)H * D * V || max_q_len <= 0)
        return NI_ERR_BAD_ARGUMENT;
    if (dtype != NI_DTYPE_F32 && dtype != NI_DTYPE_BF16) return NI_ERR_BAD_ARGUMENT;
    if (activation != 0 && activation != 1) return NI_ERR_BAD_ARGUMENT;
    if (activation == 0 && dtype != NI_DTYPE_F32) return NI_ERR_BAD_ARGUMENT;
    if (H > 65535 || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    if (max_q_len == 1) {
        dim3 grid((V + 127) / 128, H, n_seqs);
        const size_t smem = ((size_t)2 * D + (LT_THREADS / 32) * 128) * sizeof(float);
        if (smem > 48 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
        if (activation == 0)
            lightning_token_kernel<LtPlain, false><<<grid, LT_THREADS, smem, stream>>>((const LtPlain*)proj, ld, state, state_stride,
                                                                                        cu_q, slots, decay, out, H, D, V, nullptr, nullptr, 0, 1.f);
        else if (dtype == NI_DTYPE_F32)
            lightning_token_kernel<float, false><<<grid, LT_THREADS, smem, stream>>>((const float*)proj, ld, state, state_stride, cu_q,
                                                                                      slots, decay, out, H, D, V, nullptr, nullptr, 0, 1.f);
        else
            lightning_token_kernel<__nv_bfloat16, false><<<grid, LT_THREADS, smem, stream>>>(
                (const __nv_bfloat16*)proj, ld, state, state_stride, cu_q, slots, decay, out, H, D, V, nullptr, nullptr, 0, 1.f);
        NI_RETURN_LAUNCH_STATUS();
    }
    if (buf == nullptr || buf_chunks < ni_lightning_max_chunks(n_tokens, n_seqs)) return NI_ERR_BAD_ARGUMENT;
    float* before = buf + (size_t)lt_chunks(n_tokens, n_seqs) * H * D * V;      // the second half: the state before every chunk
    const int VT = D <= 128 ? 64 : 32;
    const size_t smem = lt_out_smem_bytes(D, VT);
    if (smem > 227 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
    const int per_seq = (max_q_len + LT_C - 1) / LT_C;
    const int d_tiles = (D + LT_KV_TILE - 1) / LT_KV_TILE, kv_tiles = (V + LT_KV_TILE - 1) / LT_KV_TILE, v_tiles = (V + VT - 1) / VT;
    dim3 grid_kv(per_seq * d_tiles * kv_tiles, H, n_seqs), grid_scan((D * V + LT_THREADS - 1) / LT_THREADS, H, n_seqs),
        grid_out(per_seq * v_tiles, H, n_seqs);
    const bool tc = dtype == NI_DTYPE_BF16 && D % 16 == 0 && V % 16 == 0 && ld % 8 == 0 &&
                    (reinterpret_cast<size_t>(proj) & 15) == 0 && (reinterpret_cast<size_t>(buf) & 15) == 0 &&
                    (reinterpret_cast<size_t>(out) & 7) == 0;
    if (tc) {
        const size_t smem_kv = ((size_t)2 * LT_C * (D + 8) + (size_t)LT_C * (V + 8)) * sizeof(__nv_bfloat16);
        // shared memory of the read-out kernel: q, k, the two planes of the state, and the values unless they take the keys' place
        auto out_bytes = [&](int vt) {
            return ((size_t)2 * LT_C * (D + 8) + (size_t)2 * D * (vt + 8) + (D >= vt ? 0 : (size_t)LT_C * (vt + 8))) * sizeof(__nv_bfloat16);
        };
        const int VT = V > 64 && out_bytes(128) <= 160 * 1024 ? 128 : 64;
        const int v_in_k = D >= VT;
        const size_t smem_out = out_bytes(VT);
        if (smem_kv <= 200 * 1024 && smem_out <= 200 * 1024) {
            const int vt_tiles = (V + VT - 1) / VT;
            const __nv_bfloat16* p = (const __nv_bfloat16*)proj;
            cudaFuncSetAttribute(lightning_chunk_kv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
            lightning_chunk_kv_tc_kernel<<<dim3(per_seq, H, n_seqs), LT_THREADS, smem_kv, stream>>>(p, ld, cu_q, decay, buf, H, D, V);
            lightning_scan_kernel<<<grid_scan, LT_THREADS, 0, stream>>>(state, state_stride, cu_q, slots, decay, buf, before, 1, H, D, V);
            if (VT == 128) {
                cudaFuncSetAttribute(lightning_chunk_out_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
                lightning_chunk_out_tc_kernel<128><<<dim3(per_seq * vt_tiles, H, n_seqs), 256, smem_out, stream>>>(
                    p, ld, cu_q, decay, before, out, H, D, V, vt_tiles, v_in_k);
            } else {
                cudaFuncSetAttribute(lightning_chunk_out_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
                lightning_chunk_out_tc_kernel<64><<<dim3(per_seq * vt_tiles, H, n_seqs), 128, smem_out, stream>>>(
                    p, ld, cu_q, decay, before, out, H, D, V, vt_tiles, v_in_k);
            }
            NI_RETURN_LAUNCH_STATUS();
        }
    }
#define LAUNCH(T)                                                                                                        \
    do {                                                                                                                 \
        lightning_chunk_kv_kernel<T><<<grid_kv, LT_THREADS, 0, stream>>>((const T*)proj, ld, cu_q, decay, buf, H, D, V,  \
                                                                         d_tiles, kv_tiles);                             \
        lightning_scan_kernel<<<grid_scan, LT_THREADS, 0, stream>>>(state, state_stride, cu_q, slots, decay, buf, before, 0, H, D, V); \
        if (VT == 64) {                                                                                                  \
            cudaFuncSetAttribute(lightning_chunk_out_kernel<T, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            lightning_chunk_out_kernel<T, 64><<<grid_out, LT_THREADS, smem, stream>>>((const T*)proj, ld, cu_q, decay, before, \
                                                                                      out, H, D, V, v_tiles);            \
        } else {                                                                                                         \
            cudaFuncSetAttribute(lightning_chunk_out_kernel<T, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            lightning_chunk_out_kernel<T, 32><<<grid_out, LT_THREADS, smem, stream>>>((const T*)proj, ld, cu_q, decay, before, \
                                                                                      out, H, D, V, v_tiles);            \
        }                                                                                                                \
    } while (0)
    if (activation == 0) LAUNCH(LtPlain);
    else if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else LAUNCH(__nv_bfloat16);
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}

NI_EXPORT int ni_lightning_gated_norm(const float* o, const void* proj, int dtype, int ld, int col0, const float* weight,
                                      float eps, void* y, int n_tokens, int N, cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (N <= 0 || col0 < 0 || col0 + N > ld) return NI_ERR_BAD_ARGUMENT;
    const int threads = N >= 1024 ? 256 : 128;
    if (dtype == NI_DTYPE_BF16 && N % 8 == 0 && ld % 8 == 0 && col0 % 8 == 0 && ((reinterpret_cast<size_t>(o) | reinterpret_cast<size_t>(proj) |
                                                                                  reinterpret_cast<size_t>(weight) | reinterpret_cast<size_t>(y)) & 15) == 0) {
        lightning_gated_norm_vec_kernel<<<n_tokens, N >= 2048 ? 256 : 128, 0, stream>>>(o, (const __nv_bfloat16*)proj, ld, col0, weight, eps,
                                                                                     (__nv_bfloat16*)y, N);
        NI_RETURN_LAUNCH_STATUS();
    }
#define LAUNCH(T) \
    lightning_gated_norm_kernel<T><<<n_tokens, threads, 0, stream>>>(o, (const T*)proj, ld, col0, weight, eps, (T*)y, N)
    if (dtype == NI_DTYPE_F32) LAUNCH(float);
    else if (dtype == NI_DTYPE_BF16) LAUNCH(__nv_bfloat16);
    else return NI_ERR_BAD_ARGUMENT;
#undef LAUNCH
    NI_RETURN_LAUNCH_STATUS();
}


// ---- what a retention layer puts around the recurrence ------------------------------------------------------------
//
// Retention is the same recurrence with other things before and after it: queries and keys are rotated by position
// (the first rotary_dim dimensions of every head, dimension i paired with i + rotary_dim / 2, angle = float(position)
// * inv_freq[i]), keys are then multiplied by k_scale, nothing is activated; every head's read-out is divided by its
// own root mean square and multiplied by an activation of a gate projection.

// qkv[t] = [rot(q) | rot(k) * k_scale | v] as FP32, from proj [T, ld] with columns q (H D) | k (H D) | v (H V) | ...
template <typename T>
__global__ void __launch_bounds__(256)
linear_attention_prepare_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                const float* __restrict__ inv_freq, float k_scale, float* __restrict__ qkv, int H, int D, int V,
                                int rotary_dim) {
    extern __shared__ __align__(16) float cs[];          // [rotary_dim]: cosines, then sines
    const int t = blockIdx.x, half = rotary_dim >> 1, nqk = 2 * H * D, nv = H * V;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf(pos * inv_freq[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    const T* x = proj + (size_t)t * ld;
    float* o = qkv + (size_t)t * (nqk + nv);
    for (int i = threadIdx.x; i < nqk; i += blockDim.x) {
        const int dim = i % D;
        float a = ni_to_float(x[i]);
        if (dim < rotary_dim) {
            const bool first = dim < half;
            const float b = ni_to_float(x[first ? i + half : i - half]);
            const int f = first ? dim : dim - half;
            a = first ? a * cs[f] - b * cs[half + f] : a * cs[f] + b * cs[half + f];
        }
        o[i] = i >= H * D ? a * k_scale : a;
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) o[nqk + i] = ni_to_float(x[nqk + i]);
}

NI_EXPORT int ni_linear_attention_prepare(const void* proj, int dtype, int ld, const int* positions, const float* inv_freq,
                                          float k_scale, float* qkv, int n_tokens, int H, int D, int V, int rotary_dim,
                                          cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (H <= 0 || D <= 0 || V <= 0 || rotary_dim < 0 || rotary_dim > D || (rotary_dim & 1) || ld < 2 * H * D + H * V)
        return NI_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(rotary_dim > 0 ? rotary_dim : 1) * sizeof(float);
    if (smem > 48 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
    const int threads = 2 * H * D >= 1024 ? 256 : 128;
    if (dtype == NI_DTYPE_F32)
        linear_attention_prepare_kernel<float><<<n_tokens, threads, smem, stream>>>((const float*)proj, ld, positions, inv_freq,
                                                                                    k_scale, qkv, H, D, V, rotary_dim);
    else if (dtype == NI_DTYPE_BF16)
        linear_attention_prepare_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(
            (const __nv_bfloat16*)proj, ld, positions, inv_freq, k_scale, qkv, H, D, V, rotary_dim);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// A step of single tokens of a retention layer in ONE launch: rotation, key scale, state update and read-out, straight
// from the projection (columns q (H D) | k (H D) | v (H V) | ...); every request brings one token.
NI_EXPORT int ni_retention_token_step(const void* proj, int dtype, int ld, float* state, long long state_stride,
                                      const int* cu_q, const int* slots, const float* decay, float* out, int n_seqs, int H,
                                      int D, int V, const int* positions, const float* inv_freq, int rotary_dim,
                                      float k_scale, cudaStream_t stream) {
    if (n_seqs <= 0) return NI_OK;
    if (H <= 0 || D <= 0 || V <= 0 || ld < 2 * H * D + H * V || state_stride < (long long)H * D * V || rotary_dim < 0 ||
        rotary_dim > D || (rotary_dim & 1))
        return NI_ERR_BAD_ARGUMENT;
    if (H > 65535 || n_seqs > 65535) return NI_ERR_UNSUPPORTED_SIZE;
    dim3 grid((V + 127) / 128, H, n_seqs);
    const size_t smem = ((size_t)2 * D + (LT_THREADS / 32) * 128) * sizeof(float);
    if (smem > 48 * 1024) return NI_ERR_UNSUPPORTED_SIZE;
    if (dtype == NI_DTYPE_F32)
        lightning_token_kernel<float, true><<<grid, LT_THREADS, smem, stream>>>((const float*)proj, ld, state, state_stride, cu_q,
                                                                                 slots, decay, out, H, D, V, positions, inv_freq,
                                                                                 rotary_dim, k_scale);
    else if (dtype == NI_DTYPE_BF16)
        lightning_token_kernel<__nv_bfloat16, true><<<grid, LT_THREADS, smem, stream>>>(
            (const __nv_bfloat16*)proj, ld, state, state_stride, cu_q, slots, decay, out, H, D, V, positions, inv_freq, rotary_dim,
            k_scale);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}

// y[t, g, :] = o[t, g, :] / sqrt(mean(o[t, g, :]^2) + eps) * weight[g, :] * act(gate[t, g, :]) for every group g of V
// neighbouring columns (weight null: 1), times `scale`; the gate's columns lie in proj at col0; gate_act 0: sigmoid,
// 1: silu.  One block per token, a warp takes a group at a time.
template <typename T>
__global__ void group_gated_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, int ld, int col0,
                                        const float* __restrict__ weight, float eps, T* __restrict__ y, int groups, int V,
                                        int gate_act, float scale) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const float* row = o + (size_t)t * groups * V;
    const T* g = proj + (size_t)t * ld + col0;
    T* yr = y + (size_t)t * groups * V;
    for (int grp = threadIdx.x >> 5; grp < groups; grp += warps) {
        const float* x = row + (size_t)grp * V;
        float ss = 0.f;
        for (int i = lane; i < V; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = ni_warp_sum(ss);
        const float inv = scale / sqrtf(ss / (float)V + eps);
        for (int i = lane; i < V; i += 32) {
            const int c = grp * V + i;
            const float z = ni_to_float(g[c]);
            const float sig = 1.0f / (1.0f + expf(-z));
            yr[c] = ni_from_float<T>(x[i] * inv * (weight ? weight[c] : 1.0f) * (gate_act ? z * sig : sig));
        }
    }
}

NI_EXPORT int ni_group_gated_norm(const float* o, const void* proj, int dtype, int ld, int col0, const float* weight,
                                  float eps, void* y, int n_tokens, int groups, int V, int gate_act, float scale,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return NI_OK;
    if (groups <= 0 || V <= 0 || col0 < 0 || (long long)col0 + (long long)groups * V > ld || (gate_act != 0 && gate_act != 1))
        return NI_ERR_BAD_ARGUMENT;
    const int threads = groups >= 8 ? 256 : (groups >= 4 ? 128 : 64);
    if (dtype == NI_DTYPE_F32)
        group_gated_norm_kernel<float><<<n_tokens, threads, 0, stream>>>(o, (const float*)proj, ld, col0, weight, eps, (float*)y,
                                                                         groups, V, gate_act, scale);
    else if (dtype == NI_DTYPE_BF16)
        group_gated_norm_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(o, (const __nv_bfloat16*)proj, ld, col0, weight,
                                                                                 eps, (__nv_bfloat16*)y, groups, V, gate_act, scale);
    else
        return NI_ERR_BAD_ARGUMENT;
    NI_RETURN_LAUNCH_STATUS();
}
