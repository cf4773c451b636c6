// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
// Per head, with the state S [d][dv] of a sequence (float32, zero at the sequence's start, carried from step to
// step in the cache's per-slot state):
//     S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t,
// q and k rotated (pairs (i, i + rot/2) of the first `rot` elements, by the step's cos/sin tables), k multiplied
// by `kscale` after the rotation.  Every head's o_t is then divided by its root mean square over dv (eps inside
// the root, no weight), multiplied by silu(g_t) and by `out_scale`, and stored in the compute dtype for the
// output projection.  Everything between the projections' outputs and that store is float32.
//
// Three forms of the same sums (the third, over many CTAs, is described further down):
//   * scan: tokens one after the other, the state in registers (a thread owns one column of the state and up to
//     RPT of its rows).  Decode steps, the 32-bit path, and the twin of the chunked form.
//   * chunked: a prompt's tokens in chunks of RC; inside a chunk the outputs are
//     o_i = decay^(i+1) S_in^T q_i + sum_{j<=i} decay^(i-j) (q_i . k_j) v_j and the state moves once per chunk,
//     S_out = decay^n S_in + sum_j decay^(n-1-j) k_j v_j^T.  float32 on the CUDA cores throughout.
#include "common.cuh"

#define RET_TB 8          // tokens per round of the scan form
#define RET_MAX_THREADS 512

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// Rotated q and k of `nb` tokens starting at row t0 into shared memory (float32), v beside them.
template <typename T>
__device__ __forceinline__ void ret_load_rows(const T* qkvg, int ld, int t0, int nb, int h, int H, int d, int dv,
                                              int rot, float kscale, const float* cosv, const float* sinv,
                                              float* qs, float* ks, float* vs, int j0, int ncols, int vstride,
                                              int qstride = 0) {
    const int half = rot >> 1;
    if (qstride == 0) qstride = d;
    for (int idx = threadIdx.x; idx < nb * d; idx += blockDim.x) {
        const int tt = idx / d, i = idx - tt * d;
        const T* row = qkvg + (size_t)(t0 + tt) * ld;
        const T* qp = row + h * d;
        const T* kp = row + (size_t)H * d + h * d;
        float qv, kv;
        if (i < rot) {
            const float* c = cosv + (size_t)(t0 + tt) * half;
            const float* s = sinv + (size_t)(t0 + tt) * half;
            if (i < half) {
                qv = to_f<T>(qp[i]) * c[i] - to_f<T>(qp[i + half]) * s[i];
                kv = to_f<T>(kp[i]) * c[i] - to_f<T>(kp[i + half]) * s[i];
            } else {
                const int p = i - half;
                qv = to_f<T>(qp[p]) * s[p] + to_f<T>(qp[i]) * c[p];
                kv = to_f<T>(kp[p]) * s[p] + to_f<T>(kp[i]) * c[p];
            }
        } else {
            qv = to_f<T>(qp[i]);
            kv = to_f<T>(kp[i]);
        }
        qs[tt * qstride + i] = qv;
        ks[tt * qstride + i] = kv * kscale;
    }
    for (int idx = threadIdx.x; idx < nb * ncols; idx += blockDim.x) {
        const int tt = idx / ncols, j = idx - tt * ncols;
        vs[tt * vstride + j] = to_f<T>(qkvg[(size_t)(t0 + tt) * ld + (size_t)2 * H * d + h * dv + j0 + j]);
    }
}

// grid (sequence, head, column tile); block = parts * cols threads (cols a multiple of 32): thread (part, j) owns
// the rows part*RPT .. part*RPT+RPT-1 of column j0 + j of the state.  fused != 0 (one column tile): the block
// norms, gates and stores the outputs itself; else it leaves the raw float32 outputs in `raw` [T, H*dv].
template <typename T, int RPT>
__global__ void __launch_bounds__(RET_MAX_THREADS, 1) retention_scan_kernel(
    const T* qkvg, int ld, T* out, float* raw, float* state,
    const float* cosv, const float* sinv, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
    const int* __restrict__ seq_of_token, const float* __restrict__ decay,
    int H, int d, int dv, int rot, float kscale, float eps, float out_scale, int cols, int parts, int fused) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
    const int ncols = min(cols, dv - j0);
    const int dp = parts * RPT;                // d rounded up to the threads' shares; the tail holds zeros
    float* qs = sm;                            // [RET_TB][dp]
    float* ks = qs + RET_TB * dp;              // [RET_TB][dp]
    float* vs = ks + RET_TB * dp;              // [RET_TB][cols]
    float* os = vs + RET_TB * cols;            // [RET_TB][parts][cols]
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (end <= start) return;
    if (seq_of_token[start] < 0) {             // a padding row of a replayed batch: zeros, the state untouched
        for (int t = start; t < end; ++t)
            for (int j = threadIdx.x; j < ncols; j += blockDim.x) {
                if (fused) out[(size_t)t * H * dv + h * dv + j0 + j] = from_f<T>(0.f);
                else raw[(size_t)t * H * dv + h * dv + j0 + j] = 0.f;
            }
        return;
    }
    const int part = threadIdx.x / cols, j = threadIdx.x - part * cols;
    const bool live = j < ncols;
    const int r0 = part * RPT;
    const float a = decay[h];
    float* sp = state + (((size_t)slots[b] * H + h) * d) * dv + j0 + j;
    float S[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) S[i] = (live && r0 + i < d) ? sp[(size_t)(r0 + i) * dv] : 0.f;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    if (dp > d)
        for (int idx = threadIdx.x; idx < RET_TB * (dp - d); idx += blockDim.x) {
            const int tt = idx / (dp - d), i = d + idx % (dp - d);
            qs[tt * dp + i] = 0.f;
            ks[tt * dp + i] = 0.f;
        }
    for (int t0 = start; t0 < end; t0 += RET_TB) {
        const int nb = min(RET_TB, end - t0);
        ret_load_rows<T>(qkvg, ld, t0, nb, h, H, d, dv, rot, kscale, cosv, sinv, qs, ks, vs, j0, ncols, cols, dp);
        __syncthreads();
        if (live) {
#pragma unroll 1
            for (int tt = 0; tt < nb; ++tt) {
                const float vj = vs[tt * cols + j];
                const float* kt = ks + tt * dp + r0;
                const float* qt = qs + tt * dp + r0;
                // (rows of the thread's share that lie beyond d hold zeros in k and q: no test in the loop)
                float o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int i = 0; i < RPT; i += 2) {
                    S[i] = fmaf(a, S[i], kt[i] * vj);
                    S[i + 1] = fmaf(a, S[i + 1], kt[i + 1] * vj);
                    o0 = fmaf(S[i], qt[i], o0);
                    o1 = fmaf(S[i + 1], qt[i + 1], o1);
                }
                os[(tt * parts + part) * cols + j] = o0 + o1;
            }
        }
        __syncthreads();
        for (int tt = warp; tt < nb; tt += nwarps) {
            const size_t orow = (size_t)(t0 + tt) * H * dv + h * dv + j0;
            float ss = 0.f;
            for (int c = lane; c < ncols; c += 32) {
                float o = 0.f;
                for (int p = 0; p < parts; ++p) o += os[(tt * parts + p) * cols + c];
                if (!fused) raw[orow + c] = o;
                ss = fmaf(o, o, ss);
            }
            if (fused) {
                ss = warp_sum(ss);
                const float f = out_scale / sqrtf(ss / (float)dv + eps);
                const T* gp = qkvg + (size_t)(t0 + tt) * ld + (size_t)2 * H * d + (size_t)H * dv + h * dv;
                for (int c = lane; c < ncols; c += 32) {
                    float o = 0.f;
                    for (int p = 0; p < parts; ++p) o += os[(tt * parts + p) * cols + c];
                    out[orow + c] = from_f<T>(o * f * silu_f(to_f<T>(gp[c])));
                }
            }
        }
        // the next round's loads touch qs / ks / vs only, which no thread reads after the barrier above; its
        // outputs are written after its own first barrier, when every thread has left this loop
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        if (live && r0 + i < d) sp[(size_t)(r0 + i) * dv] = S[i];
}

// out[t, h, :] = raw[t, h, :] / rms(raw[t, h, :]) * silu(g[t, h, :]) * out_scale; one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) retention_gate_kernel(const float* raw, const T* qkvg, int ld, T* out,
                                                             const int* __restrict__ seq_of_token, int ntok, int H,
                                                             int d, int dv, float eps, float out_scale) {
    pdl_launch();
    pdl_wait();
    const long long wid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (wid >= (long long)ntok * H) return;
    const int t = (int)(wid / H), h = (int)(wid - (long long)t * H);
    const float* r = raw + ((size_t)t * H + h) * dv;
    T* o = out + ((size_t)t * H + h) * dv;
    if (seq_of_token[t] < 0) {
        for (int c = lane; c < dv; c += 32) o[c] = from_f<T>(0.f);
        return;
    }
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(r[c], r[c], ss);
    ss = warp_sum(ss);
    const float f = out_scale / sqrtf(ss / (float)dv + eps);
    const T* gp = qkvg + (size_t)t * ld + (size_t)2 * H * d + (size_t)H * dv + h * dv;
    for (int c = lane; c < dv; c += 32) o[c] = from_f<T>(r[c] * f * silu_f(to_f<T>(gp[c])));
}

// ----------------------------------------------------------------------------- chunked form
// grid (sequence, head); RC tokens a chunk; 256 threads.  Shared memory holds the chunk's rotated q and k
// [RC][d], its v [RC][dv], the masked decayed scores A [RC][RC] and the state S [d][dv] (float32 throughout).
// Per chunk of n tokens (powers of the decay from a table p[i] = decay^i made once per block):
//   A[i][j] = p[i-j] (q_i . k_j) for j <= i, else 0
//   o_i     = p[i+1] (q_i^T S) + sum_j A[i][j] v_j              (raw outputs, then norm and gate as above)
//   S       = p[n] S + sum_j p[n-1-j] k_j v_j^T
#define RET_RC 32
template <typename T>
__global__ void __launch_bounds__(256) retention_chunk_kernel(
    const T* qkvg, int ld, T* out, float* state,
    const float* cosv, const float* sinv, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
    const int* __restrict__ seq_of_token, const float* __restrict__ decay,
    int H, int d, int dv, int rot, float kscale, float eps, float out_scale) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    const int b = blockIdx.x, h = blockIdx.y;
    const int dvs = dv + 1;                    // padded rows: columns of S and v are read across rows
    float* qs = sm;                            // [RC][d]
    float* ks = qs + RET_RC * d;               // [RC][d]
    float* vs = ks + RET_RC * d;               // [RC][dvs]
    float* A = vs + RET_RC * dvs;              // [RC][RC + 1]
    float* S = A + RET_RC * (RET_RC + 1);      // [d][dvs]
    float* os = S + (size_t)d * dvs;           // [RC][dvs]
    float* pw = os + RET_RC * dvs;             // [RC + 1]
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (end <= start) return;
    if (seq_of_token[start] < 0) {
        for (int t = start; t < end; ++t)
            for (int j = threadIdx.x; j < dv; j += blockDim.x) out[(size_t)t * H * dv + h * dv + j] = from_f<T>(0.f);
        return;
    }
    const float a = decay[h];
    if (threadIdx.x <= RET_RC) {
        float p = 1.f;                          // decay^i by repeated products: the scan form's own rounding
        for (int i = 0; i < (int)threadIdx.x; ++i) p *= a;
        pw[threadIdx.x] = p;
    }
    float* sp = state + (((size_t)slots[b] * H + h) * d) * dv;
    for (int idx = threadIdx.x; idx < d * dv; idx += blockDim.x) S[(idx / dv) * dvs + idx % dv] = sp[idx];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int t0 = start; t0 < end; t0 += RET_RC) {
        const int n = min(RET_RC, end - t0);
        __syncthreads();                        // the last chunk's readers of qs / ks / vs / os are done; S is whole
        ret_load_rows<T>(qkvg, ld, t0, n, h, H, d, dv, rot, kscale, cosv, sinv, qs, ks, vs, 0, dv, dvs);
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * n; idx += blockDim.x) {
            const int i = idx / n, j = idx - i * n;
            float s = 0.f;
            if (j <= i) {
                const float* qi = qs + i * d;
                const float* kj = ks + j * d;
                for (int c = 0; c < d; ++c) s = fmaf(qi[c], kj[c], s);
                s *= pw[i - j];
            }
            A[i * (RET_RC + 1) + j] = s;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
            const int i = idx / dv, c = idx - i * dv;
            float cross = 0.f;
            const float* qi = qs + i * d;
            for (int r = 0; r < d; ++r) cross = fmaf(qi[r], S[r * dvs + c], cross);
            float o = cross * pw[i + 1];
            const float* Ai = A + i * (RET_RC + 1);
            for (int j = 0; j <= i; ++j) o = fmaf(Ai[j], vs[j * dvs + c], o);
            os[i * dvs + c] = o;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < d * dv; idx += blockDim.x) {
            const int r = idx / dv, c = idx - r * dv;
            float s = S[r * dvs + c] * pw[n];
            for (int j = 0; j < n; ++j) s = fmaf(pw[n - 1 - j] * ks[j * d + r], vs[j * dvs + c], s);
            S[r * dvs + c] = s;
        }
        for (int i = warp; i < n; i += nwarps) {
            float ss = 0.f;
            for (int c = lane; c < dv; c += 32) ss = fmaf(os[i * dvs + c], os[i * dvs + c], ss);
            ss = warp_sum(ss);
            const float f = out_scale / sqrtf(ss / (float)dv + eps);
            const T* gp = qkvg + (size_t)(t0 + i) * ld + (size_t)2 * H * d + (size_t)H * dv + h * dv;
            T* op = out + (size_t)(t0 + i) * H * dv + h * dv;
            for (int c = lane; c < dv; c += 32) op[c] = from_f<T>(os[i * dvs + c] * f * silu_f(to_f<T>(gp[c])));
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < d * dv; idx += blockDim.x) sp[idx] = S[(idx / dv) * dvs + idx % dv];
}

static size_t ret_chunk_smem(int d, int dv) {
    const size_t dvs = dv + 1;
    return (2 * (size_t)RET_RC * d + 2 * RET_RC * dvs + RET_RC * (RET_RC + 1) + (size_t)d * dvs + RET_RC + 1) * sizeof(float);
}

// 1 if the chunked form takes these head sizes (its state and chunk fit one block's shared memory).
GG_API gg_retention_chunk_takes(int d, int dv) { return ret_chunk_smem(d, dv) <= 200 * 1024 ? 1 : 0; }

// qkvg [T, ld] in `dtype`: per token the q heads (H*d), the k heads (H*d), the v heads (H*dv), the gate (H*dv).
// out [T, H*dv] in `dtype`.  state float32 [slots][H][d][dv].  raw: float32 scratch [T, H*dv] (needed where the
// scan form cuts a head's columns over several blocks; may be null otherwise).  form 0: scan, 1: chunked.
GG_API gg_retention(const void* qkvg, int dtype, int ld, void* out, float* raw, float* state, const float* cosv,
                    const float* sinv, const int* cu_seqlens, const int* slots, const int* seq_of_token,
                    const float* decay, int ntok, int n_seqs, int H, int d, int dv, int rot, float kscale, float eps,
                    float out_scale, int form, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || rot < 0 || rot > d || (rot & 1) || d > 1024) return GG_ERR_ARG;
    if (form == 1) {
        const size_t smem = ret_chunk_smem(d, dv);
        if (smem > 200 * 1024) return GG_ERR_ARG;
        GG_DISPATCH_DTYPE(dtype, T,
            if (smem > 48 * 1024)
                cudaFuncSetAttribute(retention_chunk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            gg_launch(retention_chunk_kernel<T>, dim3(n_seqs, H), dim3(256), smem, stream, 1,
                (const T*)qkvg, ld, (T*)out, state, cosv, sinv, cu_seqlens, slots, seq_of_token, decay, H, d, dv, rot,
                kscale, eps, out_scale));
        return gg_last_error();
    }
    const int dvp = (dv + 31) / 32 * 32;
    // 32 rows of the state per thread keep it in registers (64 spill at 512 threads a block); 64 only where the
    // head's rows would otherwise need more parts than a block has warps
    const int rpt = (d + 31) / 32 <= RET_MAX_THREADS / 32 ? 32 : 64;
    const int parts = (d + rpt - 1) / rpt;
    int cols = RET_MAX_THREADS / parts / 32 * 32;
    if (cols <= 0) return GG_ERR_ARG;
    if (cols > dvp) cols = dvp;
    const int tiles = (dv + cols - 1) / cols;
    const int fused = tiles == 1;
    if (!fused && raw == nullptr) return GG_ERR_ARG;
    const size_t smem = ((size_t)2 * RET_TB * parts * rpt + (size_t)RET_TB * cols * (1 + parts)) * sizeof(float);
    if (smem > 200 * 1024) return GG_ERR_ARG;
#define GG_RET_SCAN(T_, R_)                                                                                          \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            cudaFuncSetAttribute(retention_scan_kernel<T_, R_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        gg_launch(retention_scan_kernel<T_, R_>, dim3(n_seqs, H, tiles), dim3(parts * cols), smem, stream, 1,          \
                  (const T_*)qkvg, ld, (T_*)out, raw, state, cosv, sinv, cu_seqlens, slots, seq_of_token, decay, H, d, \
                  dv, rot, kscale, eps, out_scale, cols, parts, fused);                                              \
    } while (0)
    GG_DISPATCH_DTYPE(dtype, T, if (rpt == 32) GG_RET_SCAN(T, 32); else GG_RET_SCAN(T, 64));
#undef GG_RET_SCAN
    int e = gg_last_error();
    if (e || fused) return e;
    const long long total = (long long)ntok * H;
    GG_DISPATCH_DTYPE(dtype, T,
        gg_launch(retention_gate_kernel<T>, dim3((unsigned)((total + 3) / 4)), dim3(128), 0, stream, 1,
                  (const float*)raw, (const T*)qkvg, ld, (T*)out, seq_of_token, ntok, H, d, dv, eps, out_scale));
    return gg_last_error();
}

// ----------------------------------------------------------------------------- chunked form over many CTAs
// The same sums as the chunked form above, cut so that every chunk of every head is a CTA of its own:
//   1. ret_chunk_state_kernel (one CTA per chunk and head): U_c = sum_j decay^(n-1-j) k_j v_j^T, what the chunk
//      adds to the state, into scratch [chunk][head][d][dv];
//   2. ret_chunk_scan_kernel (one thread per state element): walks a sequence's chunks, S_in(c+1) = decay^n S_in(c)
//      + U_c from the slot's state, leaves S_in(c) in U_c's place and the last state in the slot;
//   3. ret_chunk_out_kernel (one CTA per chunk and head): o_i = decay^(i+1) q_i^T S_in(c) + sum_{j<=i} decay^(i-j)
//      (q_i . k_j) v_j, then norm, gate and store.
// float32 on the CUDA cores; 16 x 16 threads with register tiles; head sizes up to 128 x 128.
#define RET_PC 64            // tokens per chunk
#define RET_PMAX 128         // largest d and dv

// Which (sequence, chunk) is CTA `item`?  Chunks are numbered sequence after sequence, padding rows have none.
__device__ __forceinline__ bool ret_find_chunk(int item, const int* cu_seqlens, const int* seq_of_token, int n_seqs,
                                               int& b, int& t0, int& n) {
    for (int i = 0; i < n_seqs; ++i) {
        const int a = cu_seqlens[i], e = cu_seqlens[i + 1];
        if (e <= a || seq_of_token[a] < 0) continue;
        const int nc = (e - a + RET_PC - 1) / RET_PC;
        if (item < nc) { b = i; t0 = a + item * RET_PC; n = min(RET_PC, e - t0); return true; }
        item -= nc;
    }
    return false;
}

// Rotated q (optional) and k of `n` tokens from row t0 into shared memory with row stride ds, k times kscale and
// times wk[j] (a weight per token); v with row stride dv.
template <typename T>
__device__ __forceinline__ void ret_stage(const T* qkvg, int ld, int t0, int n, int h, int H, int d, int dv, int rot,
                                          float kscale, const float* cosv, const float* sinv, float* qs, float* ks,
                                          float* vs, int ds, const float* wk, int qstride = 0, bool swizzle = false) {
    // swizzle: element i of row tt goes to column i ^ (tt & 31) of an unpadded row (d a multiple of 32): rows that
    // differ in their low five bits then read one column from different banks, as a padded row would give them
    if (qstride == 0) qstride = ds;
    const int half = rot >> 1;
    for (int idx = threadIdx.x; idx < n * d; idx += blockDim.x) {
        const int tt = idx / d, i = idx - tt * d;
        const T* row = qkvg + (size_t)(t0 + tt) * ld;
        const T* qp = row + h * d;
        const T* kp = row + (size_t)H * d + h * d;
        float qv = 0.f, kv;
        if (i < rot) {
            const float* c = cosv + (size_t)(t0 + tt) * half;
            const float* s = sinv + (size_t)(t0 + tt) * half;
            if (i < half) {
                if (qs) qv = to_f<T>(qp[i]) * c[i] - to_f<T>(qp[i + half]) * s[i];
                kv = to_f<T>(kp[i]) * c[i] - to_f<T>(kp[i + half]) * s[i];
            } else {
                const int p = i - half;
                if (qs) qv = to_f<T>(qp[p]) * s[p] + to_f<T>(qp[i]) * c[p];
                kv = to_f<T>(kp[p]) * s[p] + to_f<T>(kp[i]) * c[p];
            }
        } else {
            if (qs) qv = to_f<T>(qp[i]);
            kv = to_f<T>(kp[i]);
        }
        if (qs) qs[tt * qstride + i] = qv;
        ks[tt * ds + (swizzle ? (i ^ (tt & 31)) : i)] = kv * kscale * (wk ? wk[tt] : 1.f);
    }
    for (int idx = threadIdx.x; idx < n * dv; idx += blockDim.x) {
        const int tt = idx / dv, j = idx - tt * dv;
        vs[tt * dv + j] = to_f<T>(qkvg[(size_t)(t0 + tt) * ld + (size_t)2 * H * d + h * dv + j]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) ret_chunk_state_kernel(
    const T* qkvg, int ld, float* U, const float* cosv, const float* sinv, const int* __restrict__ cu_seqlens,
    const int* __restrict__ seq_of_token, const float* __restrict__ decay, int n_seqs, int H, int d, int dv, int rot,
    float kscale) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    int b, t0, n;
    if (!ret_find_chunk(blockIdx.x, cu_seqlens, seq_of_token, n_seqs, b, t0, n)) return;
    const int h = blockIdx.y, ds = d + 1;
    float* ks = sm;                        // [PC][ds], already times decay^(n-1-j)
    float* vs = ks + RET_PC * ds;          // [PC][dv]
    float* wk = vs + RET_PC * dv;          // [PC]
    const float a = decay[h];
    if (threadIdx.x < n) {
        float p = 1.f;
        for (int i = 0; i < n - 1 - (int)threadIdx.x; ++i) p *= a;
        wk[threadIdx.x] = p;
    }
    __syncthreads();
    ret_stage<T>(qkvg, ld, t0, n, h, H, d, dv, rot, kscale, cosv, sinv, nullptr, ks, vs, ds, wk);
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[RET_PMAX / 16][RET_PMAX / 16];
#pragma unroll
    for (int i = 0; i < RET_PMAX / 16; ++i)
#pragma unroll
        for (int j = 0; j < RET_PMAX / 16; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        float kr[RET_PMAX / 16], vc[RET_PMAX / 16];
#pragma unroll
        for (int i = 0; i < RET_PMAX / 16; ++i) {
            kr[i] = ty + 16 * i < d ? ks[j * ds + ty + 16 * i] : 0.f;
            vc[i] = tx + 16 * i < dv ? vs[j * dv + tx + 16 * i] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < RET_PMAX / 16; ++i)
#pragma unroll
            for (int c = 0; c < RET_PMAX / 16; ++c) acc[i][c] = fmaf(kr[i], vc[c], acc[i][c]);
    }
    float* up = U + ((size_t)blockIdx.x * H + h) * d * dv;
#pragma unroll
    for (int i = 0; i < RET_PMAX / 16; ++i)
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c)
            if (ty + 16 * i < d && tx + 16 * c < dv) up[(size_t)(ty + 16 * i) * dv + tx + 16 * c] = acc[i][c];
}

__global__ void __launch_bounds__(256) ret_chunk_scan_kernel(
    float* U, float* state, const int* __restrict__ cu_seqlens, const int* __restrict__ slots,
    const int* __restrict__ seq_of_token, const float* __restrict__ decay, int H, int d, int dv) {
    pdl_launch();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int e = blockIdx.z * blockDim.x + threadIdx.x;
    const int start = cu_seqlens[b], end = cu_seqlens[b + 1];
    if (e >= d * dv || end <= start || seq_of_token[start] < 0) return;
    int base = 0;
    for (int i = 0; i < b; ++i) {
        const int a0 = cu_seqlens[i], e0 = cu_seqlens[i + 1];
        if (e0 > a0 && seq_of_token[a0] >= 0) base += (e0 - a0 + RET_PC - 1) / RET_PC;
    }
    const int n_new = end - start, nch = (n_new + RET_PC - 1) / RET_PC;
    const float a = decay[h];
    float aC = 1.f;
    for (int i = 0; i < RET_PC; ++i) aC *= a;
    float* sp = state + (((size_t)slots[b] * H + h) * d) * dv + e;
    float s = *sp;
    const size_t step = (size_t)H * d * dv;
    float* up = U + ((size_t)base * H + h) * d * dv + e;
    // eight chunks' additions are asked for at once: the walk itself is a chain of dependent multiply-adds only
    for (int c0 = 0; c0 < nch; c0 += 8) {
        float u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) u[k] = c0 + k < nch ? up[(size_t)(c0 + k) * step] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < nch) {
                up[(size_t)(c0 + k) * step] = s;           // the state the chunk starts from
                const int n = min(RET_PC, n_new - (c0 + k) * RET_PC);
                float an = aC;
                if (n < RET_PC) { an = 1.f; for (int i = 0; i < n; ++i) an *= a; }
                s = fmaf(s, an, u[k]);
            }
        }
    }
    *sp = s;
}

template <typename T>
__global__ void __launch_bounds__(256, 2) ret_chunk_out_kernel(
    const T* qkvg, int ld, T* out, const float* Sin, const float* cosv, const float* sinv,
    const int* __restrict__ cu_seqlens, const int* __restrict__ seq_of_token, const float* __restrict__ decay,
    int n_seqs, int H, int d, int dv, int rot, float kscale, float eps, float out_scale) {
    pdl_launch();
    pdl_wait();
    extern __shared__ float sm[];
    int b, t0, n;
    if (!ret_find_chunk(blockIdx.x, cu_seqlens, seq_of_token, n_seqs, b, t0, n)) return;
    // Shared memory is cut so that two CTAs share an SM at 128 x 128 heads: q rows unpadded (read as broadcasts),
    // k rows unpadded with swizzled columns where d is a multiple of 32 (else padded by one), A without padding.
    const bool swz = (d & 31) == 0;
    const int h = blockIdx.y, ds = swz ? d : d + 1, wide = max(d, dv);
    float* qs = sm;                           // [PC][wide]: q rows (stride d), later the raw outputs (stride dv)
    float* ks = qs + RET_PC * wide;           // [PC][ds]
    float* vs = ks + RET_PC * ds;             // [PC][dv]
    float* A = vs + RET_PC * dv;              // [PC][PC]
    float* pw = A + RET_PC * RET_PC;          // [PC + 1]
    const float a = decay[h];
    if (threadIdx.x <= RET_PC) {
        float p = 1.f;
        for (int i = 0; i < (int)threadIdx.x; ++i) p *= a;
        pw[threadIdx.x] = p;
    }
    ret_stage<T>(qkvg, ld, t0, n, h, H, d, dv, rot, kscale, cosv, sinv, qs, ks, vs, ds, nullptr, d, swz);
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    {   // A[i][j] = decay^(i-j) (q_i . k_j) for j <= i < n, else 0
        float acc[RET_PC / 16][RET_PC / 16];
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
            for (int j = 0; j < RET_PC / 16; ++j) acc[i][j] = 0.f;
#pragma unroll 4
        for (int r = 0; r < d; ++r) {
            float qv[RET_PC / 16], kv[RET_PC / 16];
#pragma unroll
            for (int i = 0; i < RET_PC / 16; ++i) {
                qv[i] = ty + 16 * i < n ? qs[(ty + 16 * i) * d + r] : 0.f;
                kv[i] = tx + 16 * i < n ? ks[(tx + 16 * i) * ds + (swz ? (r ^ ((tx + 16 * i) & 31)) : r)] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
                for (int j = 0; j < RET_PC / 16; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
        }
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
            for (int j = 0; j < RET_PC / 16; ++j) {
                const int qi = ty + 16 * i, kj = tx + 16 * j;
                A[qi * RET_PC + kj] = (kj <= qi && qi < n) ? acc[i][j] * pw[qi - kj] : 0.f;
            }
    }
    // o[i][c]: rows i = ty + 16 a, columns c = tx + 16 b
    float o[RET_PC / 16][RET_PMAX / 16];
#pragma unroll
    for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c) o[i][c] = 0.f;
    const float* S = Sin + ((size_t)blockIdx.x * H + h) * d * dv;
#pragma unroll 4
    for (int r = 0; r < d; ++r) {
        float qv[RET_PC / 16], sv[RET_PMAX / 16];
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i) qv[i] = ty + 16 * i < n ? qs[(ty + 16 * i) * d + r] : 0.f;
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c) sv[c] = tx + 16 * c < dv ? S[(size_t)r * dv + tx + 16 * c] : 0.f;
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
            for (int c = 0; c < RET_PMAX / 16; ++c) o[i][c] = fmaf(qv[i], sv[c], o[i][c]);
    }
#pragma unroll
    for (int i = 0; i < RET_PC / 16; ++i) {
        const float f = pw[min(ty + 16 * i + 1, RET_PC)];
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c) o[i][c] *= f;
    }
    __syncthreads();                          // A is whole; every thread is done with the q rows
#pragma unroll 4
    for (int j = 0; j < n; ++j) {
        float av[RET_PC / 16], vv[RET_PMAX / 16];
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i) av[i] = A[(ty + 16 * i) * RET_PC + j];
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c) vv[c] = tx + 16 * c < dv ? vs[j * dv + tx + 16 * c] : 0.f;
#pragma unroll
        for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
            for (int c = 0; c < RET_PMAX / 16; ++c) o[i][c] = fmaf(av[i], vv[c], o[i][c]);
    }
    float* os = qs;                           // raw outputs [PC][dv]
#pragma unroll
    for (int i = 0; i < RET_PC / 16; ++i)
#pragma unroll
        for (int c = 0; c < RET_PMAX / 16; ++c)
            if (ty + 16 * i < n && tx + 16 * c < dv) os[(ty + 16 * i) * dv + tx + 16 * c] = o[i][c];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = warp; i < n; i += 8) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss = fmaf(os[i * dv + c], os[i * dv + c], ss);
        ss = warp_sum(ss);
        const float f = out_scale / sqrtf(ss / (float)dv + eps);
        const T* gp = qkvg + (size_t)(t0 + i) * ld + (size_t)2 * H * d + (size_t)H * dv + h * dv;
        T* op = out + (size_t)(t0 + i) * H * dv + h * dv;
        for (int c = lane; c < dv; c += 32) op[c] = from_f<T>(os[i * dv + c] * f * silu_f(to_f<T>(gp[c])));
    }
}

// Zero rows for the padding sequences of a replayed batch (the chunk kernels skip them).
template <typename T>
__global__ void ret_zero_padding_kernel(T* out, const int* __restrict__ seq_of_token, int ntok, int width) {
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    if (t >= ntok || seq_of_token[t] >= 0) return;
    for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)t * width + c] = from_f<T>(0.f);
}

// The many-CTA chunked form.  scratch: (ntok / 64 + n_seqs) * H * d * dv floats (a state per chunk and head).
// d, dv <= 128.
GG_API gg_retention_chunks(const void* qkvg, int dtype, int ld, void* out, float* scratch, float* state, const float* cosv,
                           const float* sinv, const int* cu_seqlens, const int* slots, const int* seq_of_token,
                           const float* decay, int ntok, int n_seqs, int H, int d, int dv, int rot, float kscale, float eps,
                           float out_scale, cudaStream_t stream) {
    if (ntok <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || H > 65535 || d <= 0 || dv <= 0 || d > RET_PMAX || dv > RET_PMAX || rot < 0 || rot > d || (rot & 1) ||
        scratch == nullptr) return GG_ERR_ARG;
    const int chunks = ntok / RET_PC + n_seqs, ds = d + 1, wide = d > dv ? d : dv;
    const size_t smem_a = ((size_t)RET_PC * (ds + dv + 1)) * sizeof(float);
    const size_t smem_c = ((size_t)RET_PC * (wide + ((d & 31) == 0 ? d : d + 1) + dv + RET_PC) + RET_PC + 1) * sizeof(float);
    GG_DISPATCH_DTYPE(dtype, T,
        if (smem_a > 48 * 1024)
            cudaFuncSetAttribute(ret_chunk_state_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        if (smem_c > 48 * 1024)
            cudaFuncSetAttribute(ret_chunk_out_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
        gg_launch(ret_chunk_state_kernel<T>, dim3(chunks, H), dim3(256), smem_a, stream, 1, (const T*)qkvg, ld, scratch,
                  cosv, sinv, cu_seqlens, seq_of_token, decay, n_seqs, H, d, dv, rot, kscale);
        gg_launch(ret_chunk_scan_kernel, dim3(n_seqs, H, (d * dv + 255) / 256), dim3(256), 0, stream, 1, scratch, state,
                  cu_seqlens, slots, seq_of_token, decay, H, d, dv);
        gg_launch(ret_chunk_out_kernel<T>, dim3(chunks, H), dim3(256), smem_c, stream, 1, (const T*)qkvg, ld, (T*)out,
                  (const float*)scratch, cosv, sinv, cu_seqlens, seq_of_token, decay, n_seqs, H, d, dv, rot, kscale, eps,
                  out_scale);
        gg_launch(ret_zero_padding_kernel<T>, dim3(ntok), dim3(128), 0, stream, 1, (T*)out, seq_of_token, ntok, H * dv));
    return gg_last_error();
}
