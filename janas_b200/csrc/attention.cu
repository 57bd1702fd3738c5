// Causal grouped-query attention over the paged cache, for prefill rows and
// decode rows alike.
//
// A row (one token of one sequence, at position pos) sees the positions
// lo..pos of its own sequence, lo = max(0, pos + 1 - window) with a window and
// 0 without.  The positions are cut into chunks of ATT_CHUNK that start at
// absolute positions; one warp computes, for one (row, KV head, chunk), the
// partial softmax of every query head of the group: the largest score m, the
// sum l of exp(score - m) and the values weighted by them.  A second kernel
// merges a row's partials in chunk order.  Both steps depend only on the row's
// own position and keys, so a row's result is the same bits whether it runs in
// a whole prompt, alone as a decoded token, or beside other sequences.
//
// This is the reference's scheme (chunks at absolute positions, partial
// (m, l, sum w v), merged in chunk order: src/llm/attention.c:27-36,870-910;
// head h uses KV head h / (heads / kv heads): :874-875; score = (q . k) *
// scale: :107-118; causal and window limits: :734-739).  Its cut-off of
// weights below exp(-80) (:574-588) is left out: such a weight is under 2e-35
// of the largest one and cannot change a float result.
#include <stdio.h>

#include "common.cuh"
#include "kernels.h"
#include "no_alloc.h"

namespace jb {

constexpr int ATT_CHUNK = 128;  // positions per partial (two pages)
constexpr int ATT_GT = 4;       // query heads a warp carries at once

template <typename T> __device__ __forceinline__ void load16(const T *p, float *out);

template <> __device__ __forceinline__ void load16<float>(const float *p, float *out)
{
    const float4 *q = reinterpret_cast<const float4 *>(p);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float4 v = q[i];
        out[4 * i + 0] = v.x;
        out[4 * i + 1] = v.y;
        out[4 * i + 2] = v.z;
        out[4 * i + 3] = v.w;
    }
}

template <> __device__ __forceinline__ void load16<bf16>(const bf16 *p, float *out)
{
    const uint4 *q = reinterpret_cast<const uint4 *>(p);
#pragma unroll
    for (int i = 0; i < 2; i++) {
        uint4 v = q[i];
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            out[8 * i + 2 * j + 0] = __uint_as_float(w[j] << 16);
            out[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}

// Scratch per (row, head, chunk index): m, l, then hd weighted values.
__host__ __device__ inline size_t part_at(size_t row, int nh, int h, int max_chunks, int ci,
                                          int hd)
{
    return ((row * nh + h) * max_chunks + ci) * (size_t)(hd + 2);
}

// LPK lanes share one key (16 values of the head each); 32 / LPK keys a step.
template <typename T, int LPK>
__global__ void __launch_bounds__(128)
attn_partial_kernel(const T *__restrict__ q, const T *__restrict__ k_cache,
                    const T *__restrict__ v_cache, const int32_t *__restrict__ row_pos,
                    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table,
                    int bt_stride, float *__restrict__ part, int row0, int n_rows, int nh, int nkv,
                    int hd, int window, float scale, int max_chunks)
{
    constexpr int KPW = 32 / LPK;
    pdl_trigger();
    pdl_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    size_t item = (size_t)blockIdx.x * 4 + warp;
    if (item >= (size_t)n_rows * max_chunks)
        return;
    int lrow = (int)(item / max_chunks), ci = (int)(item % max_chunks);
    int row = row0 + lrow;
    int kvh = blockIdx.y;
    int group = nh / nkv;
    int g0 = blockIdx.z * ATT_GT;
    int gt = min(ATT_GT, group - g0);
    int h0 = kvh * group + g0;

    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    int c = lo / ATT_CHUNK + ci;
    if (c > pos / ATT_CHUNK)
        return;
    int t0 = max(lo, c * ATT_CHUNK), t1 = min(pos, c * ATT_CHUNK + ATT_CHUNK - 1);

    int cidx = lane % LPK, ks = lane / LPK;
    bool has_dims = cidx * 16 < hd;
    const int32_t *bt = block_table + (size_t)row_seq[row] * bt_stride;

    float qv[ATT_GT][16], o[ATT_GT][16], m[ATT_GT], l[ATT_GT];
#pragma unroll
    for (int g = 0; g < ATT_GT; g++) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; j++)
            o[g][j] = qv[g][j] = 0.0f;
        if (g < gt && has_dims)
            load16<T>(q + ((size_t)row * nh + h0 + g) * hd + cidx * 16, qv[g]);
    }

    for (int base = t0; base <= t1; base += KPW) {
        int t = base + ks;
        bool valid = t <= t1;
        float kv[16];
#pragma unroll
        for (int j = 0; j < 16; j++)
            kv[j] = 0.0f;
        size_t at = 0;
        if (valid) {
            int page = bt[t / PAGE];
            at = (((size_t)page * nkv + kvh) * PAGE + (t % PAGE)) * hd + cidx * 16;
            if (has_dims)
                load16<T>(k_cache + at, kv);
        }
        float s[ATT_GT];
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            float d = 0.0f;
#pragma unroll
            for (int j = 0; j < 16; j++)
                d = fmaf(qv[g][j], kv[j], d);
#pragma unroll
            for (int off = 1; off < LPK; off <<= 1)
                d += __shfl_xor_sync(0xffffffffu, d, off);
            s[g] = d * scale;
        }
        if (valid && has_dims)
            load16<T>(v_cache + at, kv);
        if (valid) {
#pragma unroll
            for (int g = 0; g < ATT_GT; g++) {
                float mn = fmaxf(m[g], s[g]);
                float a = expf(m[g] - mn);  // 0 the first time (m = -inf)
                float p = expf(s[g] - mn);
                m[g] = mn;
                l[g] = l[g] * a + p;
#pragma unroll
                for (int j = 0; j < 16; j++)
                    o[g][j] = o[g][j] * a + p * kv[j];
            }
        }
    }

    // the 32 / LPK key groups of the warp into one
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
            float lo_ = __shfl_xor_sync(0xffffffffu, l[g], off);
            float mn = fmaxf(m[g], mo);
            float a = mn == -INFINITY ? 0.0f : expf(m[g] - mn);
            float b = mn == -INFINITY ? 0.0f : expf(mo - mn);
            l[g] = l[g] * a + lo_ * b;
            m[g] = mn;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                float oo = __shfl_xor_sync(0xffffffffu, o[g][j], off);
                o[g][j] = o[g][j] * a + oo * b;
            }
        }
    }

    if (ks == 0) {
#pragma unroll
        for (int g = 0; g < ATT_GT; g++) {
            if (g >= gt)
                continue;
            float *dst = part + part_at((size_t)lrow, nh, h0 + g, max_chunks, ci, hd);
            if (lane == 0) {
                dst[0] = m[g];
                dst[1] = l[g];
            }
            if (has_dims) {
#pragma unroll
                for (int j = 0; j < 16; j++)
                    dst[2 + cidx * 16 + j] = o[g][j];
            }
        }
    }
}

// N partials of one (row, head), fetched together, join the running (m, l, o):
// their largest maximum first, then each weighted by e^(its maximum - that), so
// that the weights do not wait for one another.  The sums run in chunk order.
template <int N>
__device__ __forceinline__ void merge_partials(const float *__restrict__ base, size_t stride,
                                               int c0, int n_chunks, int d, int hd, float &m,
                                               float &l, float &o)
{
    float mc[N], lc[N], oc[N];
#pragma unroll
    for (int u = 0; u < N; u++) {
        const float *p = base + (size_t)min(c0 + u, n_chunks - 1) * stride;
        mc[u] = p[0];
        lc[u] = p[1];
        oc[u] = d < hd ? p[2 + d] : 0.0f;
    }
    float mn = m;
#pragma unroll
    for (int u = 0; u < N; u++)
        mn = fmaxf(mn, mc[u]);
    float a = m == -INFINITY ? 0.0f : expf(m - mn);
    l *= a;
    o *= a;
#pragma unroll
    for (int u = 0; u < N; u++) {
        float w = c0 + u < n_chunks ? expf(mc[u] - mn) : 0.0f;
        l = fmaf(lc[u], w, l);
        o = fmaf(oc[u], w, o);
    }
    m = mn;
}

// One block per (row, head); thread d owns one value of the head.
template <typename T>
__global__ void attn_merge_kernel(const float *__restrict__ part,
                                  const int32_t *__restrict__ row_pos, T *__restrict__ out,
                                  int row0, int nh, int hd, int window, int max_chunks,
                                  int chunks_per_part)
{
    pdl_trigger();
    pdl_wait();
    int lrow = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    int row = row0 + lrow;
    int pos = row_pos[row];
    int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
    // a partial covers chunks_per_part chunks; max_chunks is the partials' stride
    int n_chunks = (pos / ATT_CHUNK - lo / ATT_CHUNK + chunks_per_part) / chunks_per_part;
    const float *base = part + part_at((size_t)lrow, nh, h, max_chunks, 0, hd);
    size_t stride = part_at(0, nh, 0, max_chunks, 1, hd);
    float m = -INFINITY, l = 0.0f, o = 0.0f;
    // a row with few partials fetches four at a time, one with more sixteen, one
    // with many thirty-two: most rows need one trip to memory
    if (n_chunks <= 4) {
        merge_partials<4>(base, stride, 0, n_chunks, d, hd, m, l, o);
    } else if (n_chunks <= 16) {
        merge_partials<16>(base, stride, 0, n_chunks, d, hd, m, l, o);
    } else {
        for (int c0 = 0; c0 < n_chunks; c0 += 32)
            merge_partials<32>(base, stride, c0, n_chunks, d, hd, m, l, o);
    }
    if (d < hd)
        out[((size_t)row * nh + h) * hd + d] = from_f<T>(o / l);
}

template <typename T>
static int attention_typed(const T *q, const T *k_cache, const T *v_cache, const int32_t *row_pos,
                           const int32_t *row_seq, const int32_t *block_table, int bt_stride,
                           float *part, T *out, int row0, int n_rows, int nh, int nkv, int hd,
                           int window, float scale, int max_chunks, cudaStream_t st)
{
    int lpk = 1;
    while (lpk * 16 < hd)
        lpk <<= 1;
    int group = nh / nkv;
    size_t items = (size_t)n_rows * max_chunks;
    dim3 grid((unsigned)((items + 3) / 4), nkv, (group + ATT_GT - 1) / ATT_GT);
#define JB_ATT(L)                                                                            \
    launch(attn_partial_kernel<T, L>, grid, 128, 0, st, q, k_cache, v_cache, row_pos, row_seq, \
           block_table, bt_stride, part, row0, n_rows, nh, nkv, hd, window, scale, max_chunks)
    switch (lpk) {
    case 1: JB_ATT(1); break;
    case 2: JB_ATT(2); break;
    case 4: JB_ATT(4); break;
    case 8: JB_ATT(8); break;
    case 16: JB_ATT(16); break;
    case 32: JB_ATT(32); break;
    default: return JB_EINVAL;
    }
#undef JB_ATT
    if (cudaGetLastError() != cudaSuccess)
        return JB_ELAUNCH;
    launch(attn_merge_kernel<T>, dim3(n_rows, nh), (hd + 31) / 32 * 32, 0, st, (const float *)part,
           row_pos, out, row0, nh, hd, window, max_chunks, 1);
    return launch_status();
}

}  // namespace jb

using namespace jb;

extern "C" int jb_attention_chunk() { return ATT_CHUNK; }

// Floats of scratch that n_rows rows need.
extern "C" long long jb_attention_scratch(int n_rows, int nh, int hd, int max_chunks)
{
    return (long long)part_at((size_t)n_rows, nh, 0, max_chunks, 0, hd);
}

// Rows row0 .. row0 + n_rows - 1 of the step.  q and out: [n, nh, hd]; the
// scratch holds the partials of these rows only.  max_chunks: the most chunks
// any of the rows sees.
extern "C" int jb_attention(const void *q, const void *k_cache, const void *v_cache, int dt,
                            const int32_t *row_pos, const int32_t *row_seq,
                            const int32_t *block_table, int bt_stride, float *scratch, void *out,
                            int row0, int n_rows, int nh, int nkv, int hd, int window, float scale,
                            int max_chunks, cudaStream_t st)
{
    if (n_rows <= 0)
        return JB_OK;
    if (hd % 16 || hd > 512 || hd <= 0 || nkv <= 0 || nh % nkv || max_chunks <= 0 ||
        nkv > 65535 || nh > 65535)
        return JB_EINVAL;
    if (dt == JB_F32)
        return attention_typed<float>((const float *)q, (const float *)k_cache,
                                      (const float *)v_cache, row_pos, row_seq, block_table,
                                      bt_stride, scratch, (float *)out, row0, n_rows, nh, nkv, hd,
                                      window, scale, max_chunks, st);
    if (dt == JB_BF16)
        return attention_typed<bf16>((const bf16 *)q, (const bf16 *)k_cache,
                                     (const bf16 *)v_cache, row_pos, row_seq, block_table,
                                     bt_stride, scratch, (bf16 *)out, row0, n_rows, nh, nkv, hd,
                                     window, scale, max_chunks, st);
    return JB_EINVAL;
}

// Joins partials that are already in `scratch` (written by the tensor-core
// decode kernels) for rows row0 .. row0 + n_rows - 1.  A row has one partial per
// `chunks_per_part` chunks of its range; `max_parts` partials of room per
// (row, head).
extern "C" int jb_attention_merge(const float *scratch, const int32_t *row_pos, void *out, int dt,
                                  int row0, int n_rows, int nh, int hd, int window, int max_parts,
                                  int chunks_per_part, cudaStream_t st)
{
    if (n_rows <= 0)
        return JB_OK;
    if (hd <= 0 || hd > 512 || nh <= 0 || nh > 65535 || max_parts <= 0 || chunks_per_part <= 0)
        return JB_EINVAL;
    dim3 grid(n_rows, nh);
    int threads = (hd + 31) / 32 * 32;
    if (dt == JB_F32)
        launch(attn_merge_kernel<float>, grid, threads, 0, st, scratch, row_pos, (float *)out, row0,
               nh, hd, window, max_parts, chunks_per_part);
    else if (dt == JB_BF16)
        launch(attn_merge_kernel<bf16>, grid, threads, 0, st, scratch, row_pos, (bf16 *)out, row0,
               nh, hd, window, max_parts, chunks_per_part);
    else
        return JB_EINVAL;
    return launch_status();
}

// ------------------------------------------------------ without any allocation
// See no_alloc.h.  The partial results of jb_attention_noalloc() live here.  In
// host code this name is only a stand-in for the array: the device address is
// looked up once per device below and handed to the kernels.
static __device__ __align__(256) float g_noalloc_scratch[JB_NOALLOC_SCRATCH_FLOATS];

static thread_local char t_noalloc_error[160] = "";

extern "C" const char *jb_attention_noalloc_error(void) { return t_noalloc_error; }

extern "C" int jb_attention_noalloc(const void *q, const void *k_cache, const void *v_cache,
                                    int dt, const int32_t *row_pos, const int32_t *row_seq,
                                    const int32_t *block_table, int bt_stride, void *out, int row0,
                                    int n_rows, int nh, int nkv, int hd, int window, float scale,
                                    int max_chunks, cudaStream_t st)
{
    constexpr int MAX_DEVICES = 64;
    static float *scratch_of[MAX_DEVICES];   // the array's address on each device, once known
    t_noalloc_error[0] = 0;
    if (n_rows <= 0)
        return JB_OK;
    if (nh <= 0 || hd <= 0 || max_chunks <= 0) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "sizes must be positive");
        return JB_EINVAL;
    }
    long long need = jb_attention_scratch(n_rows, nh, hd, max_chunks);
    if (need > JB_NOALLOC_SCRATCH_FLOATS) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "%d rows need %lld floats of scratch, the fixed array has %lld: "
                 "call with fewer rows", n_rows, need, (long long)JB_NOALLOC_SCRATCH_FLOATS);
        return JB_ETOOBIG;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "no current device (or beyond %d)",
                 MAX_DEVICES);
        return JB_EDEVICE;
    }
    float *scratch = scratch_of[dev];
    if (scratch == nullptr) {
        // first call on this device: the device address of the array
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            snprintf(t_noalloc_error, sizeof t_noalloc_error,
                     "cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return JB_EDEVICE;
        }
        scratch = scratch_of[dev] = (float *)p;
    }
    int rc = jb_attention(q, k_cache, v_cache, dt, row_pos, row_seq, block_table, bt_stride,
                          scratch, out, row0, n_rows, nh, nkv, hd, window, scale, max_chunks, st);
    if (rc == JB_EINVAL)
        snprintf(t_noalloc_error, sizeof t_noalloc_error,
                 "the kernel does not take these sizes or types");
    else if (rc != JB_OK)
        snprintf(t_noalloc_error, sizeof t_noalloc_error, "the launch failed");
    return rc;
}
