// Row-wise kernels: embedding gather, RMSNorm (plain, gathered, fused with the
// residual add), the activated gate of the feed-forward.
//
// The residual stream is float; the sum of squares, the scale and the product
// with the weight are computed in float.  One block works on one row and adds
// in an order that depends only on the row's width, so a row's result does not
// depend on what else is in the batch.
//
// Formulas: the reference's rms_norm, out = (x * scale) * w with
// scale = 1 / sqrtf(mean(x^2) + eps) (src/llm/model_impl.h:635-644), its
// embedding rows without scaling (src/llm/model.c:78-91), and
// SiLU(g) * u = g / (1 + e^-g) * u (src/llm/vmath.h:64-68).
#include "common.cuh"
#include "kernels.h"

namespace jb {

template <typename TT>
__global__ void embed_kernel(const TT *__restrict__ table, const int32_t *__restrict__ tokens,
                             float *__restrict__ x, int dm)
{
    pdl_trigger();
    pdl_wait();
    size_t row = blockIdx.x;
    const TT *src = table + (size_t)tokens[row] * dm;
    float *dst = x + row * dm;
    for (int i = threadIdx.x; i < dm; i += blockDim.x)
        dst[i] = to_f(src[i]);
}

// x: [n, dm] float.  delta: S stacked [n, dm] float partial sums (or null).
// When delta is given, x[row] += delta[0][row] + delta[1][row] + ... first and
// is written back.  row_idx (or null) picks the rows that are normalized; with
// it, out has one row per entry and no delta is allowed.
// EPT: values a thread holds, ceil(dm / threads); 0: any width, nothing held.
template <typename TW, typename TO, int EPT>
__global__ void rmsnorm_kernel(float *__restrict__ x, const float *__restrict__ delta, int S,
                               size_t delta_stride, const int32_t *__restrict__ row_idx,
                               const TW *__restrict__ w, TO *__restrict__ out, int dm, float eps)
{
    constexpr int KEEP = EPT > 0 ? EPT : 1;
    __shared__ float red[32];
    pdl_trigger();
    // the norm's weight does not depend on the kernel before this one
    float wv[KEEP];
    if (EPT > 0 && out != nullptr) {
#pragma unroll
        for (int u = 0; u < KEEP; u++) {
            int i = threadIdx.x + u * blockDim.x;
            wv[u] = i < dm ? to_f(w[i]) : 0.0f;
        }
    }
    pdl_wait();
    size_t orow = blockIdx.x;
    size_t row = row_idx ? (size_t)row_idx[orow] : orow;
    float *xr = x + row * dm;
    float xv[KEEP];
    float ss = 0.0f;
    if (EPT > 0) {
#pragma unroll
        for (int u = 0; u < KEEP; u++) {
            int i = threadIdx.x + u * blockDim.x;
            float v = 0.0f;
            if (i < dm) {
                v = xr[i];
                if (delta) {
                    v = add_partials(v, delta + row * dm + i, S, delta_stride);
                    xr[i] = v;
                }
            }
            xv[u] = v;
            ss = fmaf(v, v, ss);
        }
    } else {
        for (int i = threadIdx.x; i < dm; i += blockDim.x) {
            float v = xr[i];
            if (delta) {
                v = add_partials(v, delta + row * dm + i, S, delta_stride);
                xr[i] = v;
            }
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    if (out == nullptr)
        return;
    float scale = 1.0f / sqrtf(ss / (float)dm + eps);
    TO *o = out + orow * dm;
    if (EPT > 0) {
#pragma unroll
        for (int u = 0; u < KEEP; u++) {
            int i = threadIdx.x + u * blockDim.x;
            if (i < dm)
                o[i] = from_f<TO>((xv[u] * scale) * wv[u]);
        }
    } else {
        for (int i = threadIdx.x; i < dm; i += blockDim.x)
            o[i] = from_f<TO>((xr[i] * scale) * to_f(w[i]));
    }
}

// The same for many rows at once, bfloat16 output: a warp per row, eight rows a
// block, four values per lane and load.  Its sums run in another order than
// rmsnorm_kernel's, so it serves the bfloat16 path only (the 32-bit path keeps one
// order for every batch); dm must be a multiple of 4.
template <typename TW, int WPR>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(float *__restrict__ x, const float *__restrict__ delta, int S,
                    size_t delta_stride, const TW *__restrict__ w, bf16 *__restrict__ out,
                    int n, int dm, float eps)
{
    // What keeps the memory busy is how much is in flight: WPR warps share a row
    // (more of them when there are fewer rows), and each lane fetches B values of the
    // row and B of every partial sum at a time.
    constexpr int B = 4, STEP = 32 * WPR;
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    size_t row = (size_t)blockIdx.x * (8 / WPR) + warp / WPR;
    bool live = row < (size_t)n;
    if (WPR == 1 && !live)
        return;
    if (!live)
        row = (size_t)n - 1;                       // reads only; it stores nothing
    float *xr = x + row * dm;
    const float *dr = delta ? delta + row * dm : nullptr;
    int nv = dm / 4, first = (warp % WPR) * 32 + lane;
    float ss = 0.0f;
    for (int i0 = first; i0 < nv; i0 += STEP * B) {
        float4 v[B];
#pragma unroll
        for (int b = 0; b < B; b++)
            v[b] = i0 + STEP * b < nv ? load4(xr + 4 * (i0 + STEP * b))
                                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (dr) {
            for (int s = 0; s < S; s++) {
                const float *d = dr + (size_t)s * delta_stride;
                float4 t[B];
#pragma unroll
                for (int b = 0; b < B; b++)
                    t[b] = i0 + STEP * b < nv ? load4(d + 4 * (i0 + STEP * b))
                                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int b = 0; b < B; b++) {
                    v[b].x += t[b].x; v[b].y += t[b].y; v[b].z += t[b].z; v[b].w += t[b].w;
                }
            }
#pragma unroll
            for (int b = 0; b < B; b++)
                if (live && i0 + STEP * b < nv)
                    store4(xr + 4 * (i0 + STEP * b), v[b]);
        }
#pragma unroll
        for (int b = 0; b < B; b++) {
            ss = fmaf(v[b].x, v[b].x, ss);
            ss = fmaf(v[b].y, v[b].y, ss);
            ss = fmaf(v[b].z, v[b].z, ss);
            ss = fmaf(v[b].w, v[b].w, ss);
        }
    }
    ss = warp_sum(ss);
    if (WPR > 1) {
        if (lane == 0)
            red[warp] = ss;
        __syncthreads();
        ss = 0.0f;
#pragma unroll
        for (int u = 0; u < WPR; u++)
            ss += red[warp / WPR * WPR + u];
        if (!live)
            return;
    }
    float scale = 1.0f / sqrtf(ss / (float)dm + eps);
    bf16 *o = out + row * dm;
    for (int i0 = first; i0 < nv; i0 += STEP * B) {
        float4 v[B], wv[B];
#pragma unroll
        for (int b = 0; b < B; b++) {
            int c = i0 + STEP * b < nv ? 4 * (i0 + STEP * b) : 0;
            v[b] = load4(xr + c);                   // this lane wrote it: a cache hit
            wv[b] = load4(w + c);
        }
#pragma unroll
        for (int b = 0; b < B; b++)
            if (i0 + STEP * b < nv)
                store4(o + 4 * (i0 + STEP * b),
                       make_float4((v[b].x * scale) * wv[b].x, (v[b].y * scale) * wv[b].y,
                                   (v[b].z * scale) * wv[b].z, (v[b].w * scale) * wv[b].w));
    }
}

// The same for few rows, bfloat16 output: a row is shared out among the C CTAs of
// a cluster, a value (KEEP values, for very wide rows) per thread, so that all a
// row needs is fetched at once; the CTAs' sums of squares meet through
// distributed shared memory (each writes its own into every CTA) and are added
// in rank order by everyone.  Like
// rmsnorm_rows_kernel it serves the bfloat16 path only.  cols: columns per CTA.
template <typename TW, int KEEP, int C>
__global__ void __launch_bounds__(1024)
rmsnorm_cluster_kernel(float *__restrict__ x, const float *__restrict__ delta, int S,
                       size_t delta_stride, const int32_t *__restrict__ row_idx,
                       const TW *__restrict__ w, bf16 *__restrict__ out, int dm, int cols, float eps)
{
    constexpr int PB = 16 / KEEP;
    __shared__ float red[32];
    __shared__ float shares[C];        // shares[r]: written here by the CTA of rank r
    pdl_trigger();
    uint32_t rank = cluster_rank();
    size_t orow = blockIdx.x / C;
    int col[KEEP];
    float wv[KEEP], xv[KEEP];
#pragma unroll
    for (int u = 0; u < KEEP; u++) {
        int j = threadIdx.x + u * blockDim.x;
        col[u] = j < cols && (int)rank * cols + j < dm ? (int)rank * cols + j : -1;
        wv[u] = col[u] >= 0 ? to_f(w[col[u]]) : 0.0f;
    }
    pdl_wait();
    size_t row = row_idx ? (size_t)row_idx[orow] : orow;
    float *xr = x + row * dm;
#pragma unroll
    for (int u = 0; u < KEEP; u++)
        xv[u] = col[u] >= 0 ? xr[col[u]] : 0.0f;
    if (delta) {
        const float *d = delta + row * dm;
        for (int s0 = 0; s0 < S; s0 += PB) {
            float t[KEEP][PB];
#pragma unroll
            for (int u = 0; u < KEEP; u++)
#pragma unroll
                for (int b = 0; b < PB; b++)
                    t[u][b] = (s0 + b < S && col[u] >= 0)
                                  ? d[(size_t)(s0 + b) * delta_stride + col[u]] : 0.0f;
#pragma unroll
            for (int u = 0; u < KEEP; u++)
#pragma unroll
                for (int b = 0; b < PB; b++)
                    if (s0 + b < S)
                        xv[u] += t[u][b];
        }
#pragma unroll
        for (int u = 0; u < KEEP; u++)
            if (col[u] >= 0)
                xr[col[u]] = xv[u];
    }
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < KEEP; u++)
        ss = fmaf(xv[u], xv[u], ss);
    ss = block_sum(ss, red);           // every thread has the CTA's sum
    // each CTA hands its sum to all the CTAs of the cluster (itself too): one trip
    // and one barrier, after which everything is local and nobody is read any more
    if (threadIdx.x < C)
        cluster_write(&shares[rank], threadIdx.x, ss);
    cluster_arrive();
    cluster_wait();
    float tot = 0.0f;
#pragma unroll
    for (int r = 0; r < C; r++)
        tot += shares[r];
    float scale = 1.0f / sqrtf(tot / (float)dm + eps);
    bf16 *o = out + orow * dm;
#pragma unroll
    for (int u = 0; u < KEEP; u++)
        if (col[u] >= 0)
            o[col[u]] = __float2bfloat16_rn((xv[u] * scale) * wv[u]);
}

// The same for a middling number of rows, bfloat16 output: a block per row, four
// consecutive values per thread (dm <= 4096, a multiple of 4), and everything a
// thread adds fetched together, eight partial sums at a time.  Like the two
// kernels above it serves the bfloat16 path only.
template <typename TW>
__global__ void __launch_bounds__(1024)
rmsnorm_vec_kernel(float *__restrict__ x, const float *__restrict__ delta, int S,
                   size_t delta_stride, const int32_t *__restrict__ row_idx,
                   const TW *__restrict__ w, bf16 *__restrict__ out, int dm, float eps)
{
    __shared__ float red[32];
    pdl_trigger();
    int c = 4 * threadIdx.x;
    bool mine = c < dm;
    float4 wv = mine ? load4(w + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    pdl_wait();
    size_t orow = blockIdx.x;
    size_t row = row_idx ? (size_t)row_idx[orow] : orow;
    float *xr = x + row * dm;
    float4 v = mine ? load4(xr + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (delta && mine) {
        const float *d = delta + row * dm + c;
        for (int s0 = 0; s0 < S; s0 += 8) {
            float4 t[8];
#pragma unroll
            for (int b = 0; b < 8; b++)
                if (s0 + b < S)
                    t[b] = load4(d + (size_t)(s0 + b) * delta_stride);
#pragma unroll
            for (int b = 0; b < 8; b++)
                if (s0 + b < S) {
                    v.x += t[b].x; v.y += t[b].y; v.z += t[b].z; v.w += t[b].w;
                }
        }
        store4(xr + c, v);
    }
    float ss = v.x * v.x;
    ss = fmaf(v.y, v.y, ss);
    ss = fmaf(v.z, v.z, ss);
    ss = fmaf(v.w, v.w, ss);
    ss = block_sum(ss, red);
    if (!mine)
        return;
    float scale = 1.0f / sqrtf(ss / (float)dm + eps);
    store4(out + orow * dm + c, make_float4((v.x * scale) * wv.x, (v.y * scale) * wv.y,
                                            (v.z * scale) * wv.z, (v.w * scale) * wv.w));
}

// gu: S stacked [n, 2 ff] float partial sums; columns [0, ff) are the gate,
// [ff, 2 ff) the up projection.  out[n, ff] = SiLU(gate) * up.  VEC values per
// thread (4 when ff is a multiple of 4 and nothing is split, else 1).
template <typename TO, int VEC>
__global__ void swiglu_kernel(const float *__restrict__ gu, int S, size_t stride,
                              TO *__restrict__ out, int ff, size_t total)
{
    pdl_trigger();
    pdl_wait();
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= total)
        return;
    size_t row = i / ff;
    int c = (int)(i % ff);
    const float *p = gu + row * 2 * ff;
    if (VEC == 4) {
        float4 g = *reinterpret_cast<const float4 *>(p + c);
        float4 u = *reinterpret_cast<const float4 *>(p + ff + c);
        float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int e = 0; e < 4; e++)
            out[i + e] = from_f<TO>(gv[e] / (1.0f + expf(-gv[e])) * uv[e]);
    } else {
        float g = add_partials(0.0f, p + c, S, stride);
        float u = add_partials(0.0f, p + ff + c, S, stride);
        out[i] = from_f<TO>(g / (1.0f + expf(-g)) * u);
    }
}

// Threads of a block that works on one row: about eight values each.  The
// number depends on the row's width alone, because the order in which a row's
// squares are added depends on it and a row's result must not depend on the
// batch it is in.
static int norm_threads(int dm)
{
    int t = 32;
    while (t < 1024 && t * 8 < dm)
        t <<= 1;
    return t;
}

}  // namespace jb

using namespace jb;

// Positions a page of the cache holds, as the kernels were compiled; the host side
// checks its own number against it when an engine is made.
extern "C" int jb_page(void) { return PAGE; }

extern "C" int jb_embed(const void *table, int table_dt, const int32_t *tokens, float *x, int n,
                        int dm, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    int threads = norm_threads(dm);
    if (table_dt == JB_F32)
        launch(embed_kernel<float>, n, threads, 0, st, (const float *)table, tokens, x, dm);
    else if (table_dt == JB_BF16)
        launch(embed_kernel<bf16>, n, threads, 0, st, (const bf16 *)table, tokens, x, dm);
    else
        return JB_EINVAL;
    return launch_status();
}

extern "C" int jb_rmsnorm(float *x, const float *delta, int S, long long delta_stride,
                          const int32_t *row_idx, const void *w, int w_dt, void *out, int out_dt,
                          int n_out, int dm, float eps, cudaStream_t st)
{
    if (n_out <= 0)
        return JB_OK;
    if (delta && row_idx)
        return JB_EINVAL;
    // many rows of the bfloat16 path: the kernel that takes eight rows a block
    if (out != nullptr && out_dt == JB_BF16 && row_idx == nullptr && n_out >= 256 && dm % 4 == 0 &&
        (uintptr_t)x % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)out % 8 == 0 &&
        (uintptr_t)w % (w_dt == JB_F32 ? 16 : 8) == 0 &&
        (delta == nullptr || delta_stride % 4 == 0)) {
        // enough warps to keep every SM's memory pipeline full: four per row below
        // 4,096 rows, two below 8,192, else one
        int wpr = n_out < 4096 ? 4 : n_out < 8192 ? 2 : 1;
        unsigned blocks = (unsigned)((n_out + 8 / wpr - 1) / (8 / wpr));
#define JB_NORM_R(TW, W)                                                                      \
    launch(rmsnorm_rows_kernel<TW, W>, blocks, 256, 0, st, x, delta, S, (size_t)delta_stride,  \
           (const TW *)w, (bf16 *)out, n_out, dm, eps)
#define JB_NORM_RW(TW)                                                                        \
    do {                                                                                       \
        if (wpr == 4)                                                                          \
            JB_NORM_R(TW, 4);                                                                  \
        else if (wpr == 2)                                                                     \
            JB_NORM_R(TW, 2);                                                                  \
        else                                                                                   \
            JB_NORM_R(TW, 1);                                                                  \
    } while (0)
        if (w_dt == JB_F32)
            JB_NORM_RW(float);
        else if (w_dt == JB_BF16)
            JB_NORM_RW(bf16);
        else
            return JB_EINVAL;
#undef JB_NORM_R
#undef JB_NORM_RW
        return launch_status();
    }
    // few rows of the bfloat16 path: a cluster of eight CTAs per row (measured: faster
    // than a block per row at 1 and 8 rows, slower at 64)
    if (out != nullptr && out_dt == JB_BF16 && n_out <= 32 && dm >= 1024 && dm <= 8 * 4 * 1024 &&
        (w_dt == JB_F32 || w_dt == JB_BF16)) {
        constexpr int C = 8;
        int cols = (dm + C - 1) / C;
        int keep = cols <= 1024 ? 1 : cols <= 2048 ? 2 : 4;
        unsigned threads = (unsigned)(((cols + keep - 1) / keep + 31) / 32 * 32);
        dim3 grid((unsigned)n_out * C);
#define JB_NORM_C(TW, K)                                                                      \
    launch_cluster(rmsnorm_cluster_kernel<TW, K, C>, grid, threads, 0, st, C, x, delta, S,     \
                   (size_t)delta_stride, row_idx, (const TW *)w, (bf16 *)out, dm, cols, eps)
#define JB_NORM_CK(TW)                                                                        \
    do {                                                                                       \
        if (keep == 1)                                                                         \
            JB_NORM_C(TW, 1);                                                                  \
        else if (keep == 2)                                                                    \
            JB_NORM_C(TW, 2);                                                                  \
        else                                                                                   \
            JB_NORM_C(TW, 4);                                                                  \
    } while (0)
        if (w_dt == JB_F32)
            JB_NORM_CK(float);
        else
            JB_NORM_CK(bf16);
#undef JB_NORM_C
#undef JB_NORM_CK
        return launch_status();
    }
    // a middling number of rows of the bfloat16 path: four values per thread
    if (out != nullptr && out_dt == JB_BF16 && n_out > 32 && dm % 4 == 0 && dm <= 4096 &&
        (w_dt == JB_F32 || w_dt == JB_BF16) && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)delta % 16 == 0 && (uintptr_t)out % 8 == 0 &&
        (uintptr_t)w % (w_dt == JB_F32 ? 16 : 8) == 0 && (delta == nullptr || delta_stride % 4 == 0)) {
        unsigned threads = (unsigned)((dm / 4 + 31) / 32 * 32);
        if (w_dt == JB_F32)
            launch(rmsnorm_vec_kernel<float>, n_out, threads, 0, st, x, delta, S,
                   (size_t)delta_stride, row_idx, (const float *)w, (bf16 *)out, dm, eps);
        else
            launch(rmsnorm_vec_kernel<bf16>, n_out, threads, 0, st, x, delta, S,
                   (size_t)delta_stride, row_idx, (const bf16 *)w, (bf16 *)out, dm, eps);
        return launch_status();
    }
    int threads = norm_threads(dm);
    int ept = (dm + threads - 1) / threads;
#define JB_NORM_E(TW, TO, E)                                                                  \
    launch(rmsnorm_kernel<TW, TO, E>, n_out, threads, 0, st, x, delta, S,                      \
           (size_t)delta_stride, row_idx, (const TW *)w, (TO *)out, dm, eps)
#define JB_NORM(TW, TO)                                                                       \
    do {                                                                                       \
        switch (ept) {                                                                         \
        case 1: JB_NORM_E(TW, TO, 1); break;                                                   \
        case 2: JB_NORM_E(TW, TO, 2); break;                                                   \
        case 3: JB_NORM_E(TW, TO, 3); break;                                                   \
        case 4: JB_NORM_E(TW, TO, 4); break;                                                   \
        case 5: JB_NORM_E(TW, TO, 5); break;                                                   \
        case 6: JB_NORM_E(TW, TO, 6); break;                                                   \
        case 7: JB_NORM_E(TW, TO, 7); break;                                                   \
        case 8: JB_NORM_E(TW, TO, 8); break;                                                   \
        default: JB_NORM_E(TW, TO, 0); break;                                                  \
        }                                                                                      \
    } while (0)
    if (out == nullptr)
        JB_NORM(float, float);
    else if (w_dt == JB_F32 && out_dt == JB_F32)
        JB_NORM(float, float);
    else if (w_dt == JB_F32 && out_dt == JB_BF16)
        JB_NORM(float, bf16);
    else if (w_dt == JB_BF16 && out_dt == JB_F32)
        JB_NORM(bf16, float);
    else if (w_dt == JB_BF16 && out_dt == JB_BF16)
        JB_NORM(bf16, bf16);
    else
        return JB_EINVAL;
#undef JB_NORM_E
#undef JB_NORM
    return launch_status();
}

extern "C" int jb_swiglu(const float *gu, int S, long long stride, void *out, int out_dt, int n,
                         int ff, cudaStream_t st)
{
    size_t total = (size_t)n * ff;
    if (total == 0)
        return JB_OK;
    bool vec = S == 1 && ff % 4 == 0 && (uintptr_t)gu % 16 == 0;
    size_t threads = vec ? total / 4 : total;
    unsigned blocks = (unsigned)((threads + 255) / 256);
    if (out_dt == JB_F32 && vec)
        launch(swiglu_kernel<float, 4>, blocks, 256, 0, st, gu, S, (size_t)stride, (float *)out, ff, total);
    else if (out_dt == JB_F32)
        launch(swiglu_kernel<float, 1>, blocks, 256, 0, st, gu, S, (size_t)stride, (float *)out, ff, total);
    else if (out_dt == JB_BF16 && vec)
        launch(swiglu_kernel<bf16, 4>, blocks, 256, 0, st, gu, S, (size_t)stride, (bf16 *)out, ff, total);
    else if (out_dt == JB_BF16)
        launch(swiglu_kernel<bf16, 1>, blocks, 256, 0, st, gu, S, (size_t)stride, (bf16 *)out, ff, total);
    else
        return JB_EINVAL;
    return launch_status();
}
