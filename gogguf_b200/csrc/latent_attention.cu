// Latent attention over a paged cache of one vector per position.
//
// A layer of this kind caches, per position, a latent c (R elements, RMS-normed) and one rotated key part
// k_r (r elements) that all heads share: the row [c | k_r] of the pool.  Per head h the key is
// [W_uk,h c | k_r] and the value W_uv,h c.  Because both are linear in c, a query never needs them:
//
//   score(i, j) = scale * ( (W_uk,h^T q_plain,i) . c_j  +  q_rot,i . k_r,j )
//   out_h(i)    = W_uv,h * sum_j p(i, j) c_j
//
// so a step runs   prep (norm, rotation, cache write)  ->  absorb (q_lat = W_uk,h^T q_plain, a product per head)
// ->  attention over the rows of the pool with queries [q_lat | q_rot] of R + r elements, whose weighted sum of
// the rows' first R elements is the latent output  ->  expand (W_uv,h on the latent output, a product per head).
// Every head reads the same rows: one pass over a window of the cache serves all heads, in a prompt and in
// decoding alike, and the result does not depend on how a prompt was cut into steps.
//
// Kernels here: latent_prep, headwise_gemm (the per-head products, CUDA cores, any dtype mix),
// latent_attention_plain (one block per token and head, float32 arithmetic: the 32-bit path and the twin of
// the tensor-core kernel), and latent_attention_mma (bfloat16, mma.sync, 64 query rows per CTA).
// Scores, softmax, the norm and the rotation are float32 in all of them.
#include "common.cuh"

// ----------------------------------------------------------------------------- prep
// One block per token.  dkv[t] = [latent (R) | key part (r)] as the down projection left it; q[t] holds H heads
// of [plain (d) | rot (r)].  Writes pool row [rms(latent) * w | rotate(key part)] and qcat[t, h, R : R + r] =
// rotate(q rot part).  The rotation pairs element 2i with 2i+1 for i < dims / 2 and leaves the rest as it is;
// cos/sin[t, i] are the step's tables.  Padding tokens (seq_of_token < 0) write zeros to qcat and no cache.
template <typename T, typename TQ>
__global__ void __launch_bounds__(256) latent_prep_kernel(
    const T* q, long long ldq, const T* dkv, long long lddkv, const float* __restrict__ normw, float eps,
    const float* cosv, const float* sinv, int dims, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int page_size,
    T* pool, int pool_row, TQ* qcat, int H, int d, int r, int R, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    const int half = dims >> 1;
    TQ* qc = qcat + (size_t)t * H * (R + r);
    if (b < 0) {
        for (int i = threadIdx.x; i < H * r; i += blockDim.x) qc[(size_t)(i / r) * (R + r) + R + (i % r)] = from_f<TQ>(0.f);
        return;
    }
    const float* cs = cosv + (size_t)t * half;
    const float* sn = sinv + (size_t)t * half;
    // rotated part of every query head
    const T* qt = q + (size_t)t * ldq;
    for (int i = threadIdx.x; i < H * r; i += blockDim.x) {
        const int h = i / r, e = i % r;
        const T* src = qt + (size_t)h * (d + r) + d;
        float v = to_f<T>(src[e]);
        if (e < dims) {
            const float o = to_f<T>(src[e ^ 1]);
            const float c = cs[e >> 1], s = sn[e >> 1];
            v = (e & 1) ? v * c + o * s : v * c - o * s;
        }
        qc[(size_t)h * (R + r) + R + e] = from_f<TQ>(v);
    }
    if (pool == nullptr) return;
    const T* dk = dkv + (size_t)t * lddkv;
    float ss = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = to_f<T>(dk[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float f = 1.0f / sqrtf(ss / (float)R + eps);
    const int pos = positions[t];
    const int page = gg_page_w(page_table + (size_t)b * max_pages, pos / page_size, max_pages, pb, 49);
    if (page < 0) return;
    T* row = pool + ((size_t)page * page_size + (pos % page_size)) * pool_row;
    for (int i = threadIdx.x; i < R; i += blockDim.x) row[i] = from_f<T>(to_f<T>(dk[i]) * f * normw[i]);
    for (int e = threadIdx.x; e < r; e += blockDim.x) {
        float v = to_f<T>(dk[R + e]);
        if (e < dims) {
            const float o = to_f<T>(dk[R + (e ^ 1)]);
            const float c = cs[e >> 1], s = sn[e >> 1];
            v = (e & 1) ? v * c + o * s : v * c - o * s;
        }
        row[R + e] = from_f<T>(v);
    }
}

// q, dkv and the pool share `dtype`; qcat has `q_dtype`.  pool may be null (a layer that reads another's cache).
GG_API gg_latent_prep(const void* q, long long ldq, const void* dkv, long long lddkv, int dtype, const float* normw,
                      float eps, const float* cosv, const float* sinv, int dims, const int* positions,
                      const int* seq_of_token, const int* page_table, int max_pages, int page_size, int n_pages,
                      void* pool, int pool_row, void* qcat, int q_dtype, int ntok, int H, int d, int r, int R,
                      int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || d <= 0 || r <= 0 || R <= 0 || dims < 0 || dims > r || (dims & 1) || pool_row < R + r || page_size <= 0)
        return GG_ERR_ARG;
    const PageBounds pb{n_pages, status};
#define GG_PREP(T, TQ) gg_launch(latent_prep_kernel<T, TQ>, dim3(ntok), dim3(256), 0, stream, 1, (const T*)q, ldq, \
        (const T*)dkv, lddkv, normw, eps, cosv, sinv, dims, positions, seq_of_token, page_table, max_pages, page_size, \
        (T*)pool, pool_row, (TQ*)qcat, H, d, r, R, pb)
    if (dtype == GG_F32 && q_dtype == GG_F32) GG_PREP(float, float);
    else if (dtype == GG_BF16 && q_dtype == GG_F32) GG_PREP(bf16, float);
    else if (dtype == GG_BF16 && q_dtype == GG_BF16) GG_PREP(bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_PREP
    return gg_last_error();
}

// ----------------------------------------------------------------------------- per-head products
// out[t, h, n] = alpha * sum_k x[t, h, k] * w[h, n, k] for h < H: H small products that share the token axis.
// x[t, h, k] is at x + t * ldx + h * hx + k, out[t, h, n] at out + t * ldo + h * ho + n, w[h] is [N, K] row-major.
// The sum over k runs in a fixed order that does not depend on the number of tokens.
#define HB 64
#define HK 16
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256) headwise_gemm_kernel(const TX* x, long long ldx, long long hx,
                                                            const TW* __restrict__ w, TO* out, long long ldo,
                                                            long long ho, int M, int N, int K, float alpha) {
    pdl_launch();
    pdl_wait();
    __shared__ float xs[HK][HB + 1];
    __shared__ float ws[HK][HB + 1];
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * HB, n0 = blockIdx.x * HB;
    const int tid = threadIdx.x;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    const TX* xh = x + (size_t)h * hx;
    const TW* wh = w + (size_t)h * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int rr = idx / HK, kk = idx % HK;
            const int gk = k0 + kk;
            float xv = 0.f, wv = 0.f;
            if (gk < K) {
                if (m0 + rr < M) xv = to_f<TX>(xh[(size_t)(m0 + rr) * ldx + gk]);
                if (n0 + rr < N) wv = to_f<TW>(wh[(size_t)(n0 + rr) * K + gk]);
            }
            xs[kk][rr] = xv;
            ws[kk][rr] = wv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HK; ++kk) {
            float a[4], bq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bq[j] = ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bq[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) out[(size_t)m * ldo + (size_t)h * ho + n] = from_f<TO>(acc[i][j] * alpha);
        }
    }
}

GG_API gg_headwise_gemm(const void* x, int x_dtype, long long ldx, long long hx, const void* w, int w_dtype,
                        void* out, int out_dtype, long long ldo, long long ho, int M, int N, int K, int H,
                        float alpha, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || H <= 0) return 0;
    if (K <= 0 || H > 65535 || (M + HB - 1) / HB > 65535) return GG_ERR_ARG;
    dim3 grid((N + HB - 1) / HB, (M + HB - 1) / HB, H);
#define GG_HW(TX, TW, TO) gg_launch(headwise_gemm_kernel<TX, TW, TO>, dim3(grid), dim3(256), 0, stream, 1, \
        (const TX*)x, ldx, hx, (const TW*)w, (TO*)out, ldo, ho, M, N, K, alpha)
    const int code = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (code) {
        case 0: GG_HW(float, float, float); break;
        case 1: GG_HW(float, float, bf16); break;
        case 2: GG_HW(float, bf16, float); break;
        case 3: GG_HW(float, bf16, bf16); break;
        case 4: GG_HW(bf16, float, float); break;
        case 5: GG_HW(bf16, float, bf16); break;
        case 6: GG_HW(bf16, bf16, float); break;
        case 7: GG_HW(bf16, bf16, bf16); break;
        default: return GG_ERR_DTYPE;
    }
#undef GG_HW
    return gg_last_error();
}

// ----------------------------------------------------------------------------- attention, plain
// One block per (token, head).  The token at position p of sequence b reads the pool rows of positions lo..p,
// lo = max(0, p - window + 1) for a windowed layer (itself included: its row was written by latent_prep).
#define LAT_WARPS 4
#define LAT_MAXR 1024

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(LAT_WARPS * 32) latent_attention_plain_kernel(
    const TQ* qcat, const TC* pool, int pool_row, TO* out, const int* __restrict__ positions,
    const int* __restrict__ seq_of_token, const int* __restrict__ page_table, int max_pages, int page_size,
    int H, int R, int r, float scale, int window, const PageBounds pb) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int D = R + r;
    float* qs = sm;                       // [D]
    float* accs = sm + D;                 // [LAT_WARPS][R]
    float* ml = accs + LAT_WARPS * R;     // [LAT_WARPS][2]
    const int t = blockIdx.x, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TO* o = out + ((size_t)t * H + h) * R;
    const int b = seq_of_token[t];
    if (b < 0) {
        for (int i = threadIdx.x; i < R; i += blockDim.x) o[i] = from_f<TO>(0.f);
        return;
    }
    const int pos = positions[t];
    int lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    const TQ* qp = qcat + ((size_t)t * H + h) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) qs[i] = to_f<TQ>(qp[i]);
    __syncthreads();
    float acc[LAT_MAXR / 32];
#pragma unroll
    for (int j = 0; j < LAT_MAXR / 32; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int* pt = page_table + (size_t)b * max_pages;
    for (int j = lo + warp; j <= pos; j += LAT_WARPS) {
        const int page = gg_page(pt, j / page_size, max_pages, pb, 50);
        const TC* row = pool + ((size_t)page * page_size + (j % page_size)) * pool_row;
        float dot = 0.f;
        for (int i = lane; i < D; i += 32) dot = fmaf(qs[i], to_f<TC>(row[i]), dot);
        dot = warp_sum(dot) * scale;
        const float mn = fmaxf(m, dot);
        const float corr = expf(m - mn);
        const float p = expf(dot - mn);
        l = l * corr + p;
#pragma unroll
        for (int jj = 0; jj < LAT_MAXR / 32; ++jj) {
            const int i = lane + 32 * jj;
            if (i < R) acc[jj] = acc[jj] * corr + p * to_f<TC>(row[i]);
        }
        m = mn;
    }
#pragma unroll
    for (int jj = 0; jj < LAT_MAXR / 32; ++jj) {
        const int i = lane + 32 * jj;
        if (i < R) accs[warp * R + i] = acc[jj];
    }
    if (lane == 0) { ml[warp * 2] = m; ml[warp * 2 + 1] = l; }
    __syncthreads();
    float Mx = -INFINITY;
    for (int w = 0; w < LAT_WARPS; ++w) Mx = fmaxf(Mx, ml[w * 2]);
    float L = 0.f;
    float f[LAT_WARPS];
    for (int w = 0; w < LAT_WARPS; ++w) {
        f[w] = ml[w * 2] == -INFINITY ? 0.f : expf(ml[w * 2] - Mx);
        L += ml[w * 2 + 1] * f[w];
    }
    const float inv = 1.0f / L;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < LAT_WARPS; ++w) s += accs[w * R + i] * f[w];
        o[i] = from_f<TO>(s * inv);
    }
}

// qcat [T, H, R + r] in q_dtype, pool [page][page_size][pool_row] in c_dtype, out [T, H, R] in o_dtype.
GG_API gg_latent_attention_plain(const void* qcat, int q_dtype, const void* pool, int c_dtype, int pool_row, void* out,
                                 int o_dtype, const int* positions, const int* seq_of_token, const int* page_table,
                                 int max_pages, int page_size, int n_pages, int ntok, int H, int R, int r, float scale,
                                 int window, int* status, cudaStream_t stream) {
    if (ntok <= 0) return 0;
    if (H <= 0 || H > 65535 || R <= 0 || R > LAT_MAXR || r < 0 || pool_row < R + r || page_size <= 0) return GG_ERR_ARG;
    const size_t smem = ((size_t)(R + r) + (size_t)LAT_WARPS * R + 2 * LAT_WARPS) * sizeof(float);
    if (smem > 48 * 1024) return GG_ERR_ARG;
    const PageBounds pb{n_pages, status};
    dim3 grid(ntok, H);
#define GG_LAP(TQ, TC, TO) gg_launch(latent_attention_plain_kernel<TQ, TC, TO>, dim3(grid), dim3(LAT_WARPS * 32), smem, \
        stream, 1, (const TQ*)qcat, (const TC*)pool, pool_row, (TO*)out, positions, seq_of_token, page_table, max_pages, \
        page_size, H, R, r, scale, window, pb)
    if (q_dtype == GG_F32 && c_dtype == GG_F32 && o_dtype == GG_F32) GG_LAP(float, float, float);
    else if (q_dtype == GG_F32 && c_dtype == GG_BF16 && o_dtype == GG_F32) GG_LAP(float, bf16, float);
    else if (q_dtype == GG_BF16 && c_dtype == GG_BF16 && o_dtype == GG_BF16) GG_LAP(bf16, bf16, bf16);
    else return GG_ERR_DTYPE;
#undef GG_LAP
    return gg_last_error();
}

GG_API gg_latent_attention_checked() { return gg_debug_bounds(); }
