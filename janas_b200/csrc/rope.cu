// Position encoding: the RoPE table, and the fused per-head q/k RMSNorm +
// NeoX rotation + append of K and V to the paged cache.
//
// Formulas (reference): theta(p, i) = (float)p * inv_freq[i] with
// inv_freq[i] = powf(base, -2 i / n_rot) (src/llm/model.c:100-113), cos and
// sin evaluated in double and rounded once (src/llm/jmath.c:163-200); per head
// RMSNorm with one weight vector for all heads, before the rotation
// (src/llm/model_attn.c:93-101); pairs (i, i + half):
// v[i] = a cos - b sin, v[i + half] = a sin + b cos
// (src/llm/model_attn.c:31-39); K after norm and rotation and V as it is go to
// the cache at the row's position (src/llm/model_attn.c:103-145; the
// reference's eight-bit cache is not reproduced).
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace jb {

__global__ void rope_table_kernel(float *__restrict__ cs, float *__restrict__ sn,
                                  const float *__restrict__ inv_freq, int n_pos, int half)
{
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_pos * half)
        return;
    int p = (int)(i / half), f = (int)(i % half);
    float theta = __fmul_rn((float)p, inv_freq[f]);
    double s, c;
    sincos((double)theta, &s, &c);
    cs[i] = (float)c;
    sn[i] = (float)s;
}

// One warp per (row, head slot); head slots are the q heads, then the k heads,
// then the v heads of the row's fused [q | k | v] vector.  PAIRS is how many
// (low, high) pairs of a head a lane holds: ceil(hd / 64).  This kernel takes
// every even head size up to 512; the usual sizes go to the kernel below.
//
// qkv: S stacked [n, (nh + 2 nkv) hd] float partial sums.
// q_out: [n, nh, hd] in the cache's type.  K and V go to page
// block_table[seq][pos / PAGE] of k_cache / v_cache, which are laid out
// [page][kv head][PAGE][hd].
template <typename TC, typename TW, int PAIRS>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_kernel(
    const float *__restrict__ qkv, int S, size_t split_stride, const TW *__restrict__ q_w,
    const TW *__restrict__ k_w, float eps, const float *__restrict__ cs,
    const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table, int bt_stride,
    TC *__restrict__ q_out, TC *__restrict__ k_cache, TC *__restrict__ v_cache, int n, int nh,
    int nkv, int hd)
{
    pdl_trigger();
    unsigned slots = nh + 2 * nkv;
    unsigned task = blockIdx.x * blockDim.y + threadIdx.y;
    if (task >= (unsigned)n * slots)
        return;
    unsigned row = task / slots, hs = task - row * slots;
    int lane = threadIdx.x;
    int half = hd / 2;
    bool is_q = hs < (unsigned)nh;
    bool is_v = hs >= (unsigned)(nh + nkv);

    // Positions, page tables, rotation tables and norm weights were written long
    // before the kernel before this one: they are fetched before the wait.
    int pos = row_pos[row];
    int page = k_cache != nullptr
                   ? block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE] : 0;
    bool normed = !is_v && q_w != nullptr;
    bool rotate = !is_v && rot_half == half;
    const TW *w = is_q ? q_w : k_w;
    float co[PAIRS], si[PAIRS], wl[PAIRS], wh[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        int i = lane + 32 * j;
        co[j] = 1.0f;
        si[j] = 0.0f;
        wl[j] = wh[j] = 1.0f;
        if (i < half) {
            if (rotate) {
                co[j] = cs[(size_t)pos * rot_half + i];
                si[j] = sn[(size_t)pos * rot_half + i];
            }
            if (normed) {
                wl[j] = to_f(w[i]);
                wh[j] = to_f(w[i + half]);
            }
        }
    }
    pdl_wait();

    TC *dst;
    if (is_q) {
        dst = q_out + ((size_t)row * nh + hs) * hd;
    } else {
        if (k_cache == nullptr)
            return;
        int kvh = !is_v ? hs - nh : hs - nh - nkv;
        size_t at = (((size_t)page * nkv + kvh) * PAGE + (pos % PAGE)) * hd;
        dst = (!is_v ? k_cache : v_cache) + at;
    }
    const float *src = qkv + (size_t)row * slots * hd + (size_t)hs * hd;
    float lo[PAIRS], hi[PAIRS];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        int i = lane + 32 * j;
        lo[j] = hi[j] = 0.0f;
        if (i < half) {
            lo[j] = add_partials(0.0f, src + i, S, split_stride);
            hi[j] = add_partials(0.0f, src + i + half, S, split_stride);
        }
        ss = fmaf(lo[j], lo[j], ss);
        ss = fmaf(hi[j], hi[j], ss);
    }
    float scale = 1.0f;
    if (normed) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + eps);
    }
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        int i = lane + 32 * j;
        if (i < half) {
            float a = lo[j], b = hi[j];
            if (normed) {
                a = (a * scale) * wl[j];
                b = (b * scale) * wh[j];
            }
            if (rotate) {
                dst[i] = from_f<TC>(a * co[j] - b * si[j]);
                dst[i + half] = from_f<TC>(a * si[j] + b * co[j]);
            } else {
                dst[i] = from_f<TC>(a);
                dst[i + half] = from_f<TC>(b);
            }
        }
    }
}

// The same for head sizes 32, 64, 128 and 256: LPH = hd / 8 lanes share a head
// slot, each with four consecutive values of the low half and the four that
// pair with them in the high half, so that a warp works on 32 / LPH head slots
// of its row at once with 16-byte loads.  Everything must lie on 16-byte
// boundaries (the launcher checks).  The sums of squares are added in another
// order than in the kernel above; which of the two runs depends on the head
// size and the addresses only, never on the number of rows.
template <typename TC, typename TW, int LPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_vec_kernel(
    const float *__restrict__ qkv, int S, size_t split_stride, const TW *__restrict__ q_w,
    const TW *__restrict__ k_w, float eps, const float *__restrict__ cs,
    const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table, int bt_stride,
    TC *__restrict__ q_out, TC *__restrict__ k_cache, TC *__restrict__ v_cache, int n, int nh,
    int nkv)
{
    constexpr int SLOTS_PER_WARP = 32 / LPH;
    constexpr int half = 4 * LPH, hd = 2 * half;
    pdl_trigger();
    unsigned slots = nh + 2 * nkv;
    unsigned groups = (slots + SLOTS_PER_WARP - 1) / SLOTS_PER_WARP;
    unsigned total = (unsigned)n * groups;
    int at4 = 4 * (threadIdx.x % LPH);          // this lane's values: at4 .. at4 + 3 of each half
    bool waited = false;
    // with many rows a warp takes several tasks in turn: blocks that live for one
    // task only are started more slowly than they finish
    for (unsigned task = blockIdx.x * blockDim.y + threadIdx.y; task < total;
         task += gridDim.x * blockDim.y) {
        unsigned row = task / groups;
        unsigned hs = (task - row * groups) * SLOTS_PER_WARP + threadIdx.x / LPH;
        bool live = hs < slots;
        bool is_q = hs < (unsigned)nh;
        bool is_v = hs >= (unsigned)(nh + nkv);

        // positions, page tables, rotation tables and norm weights were written long
        // before the kernel before this one: they are fetched before the wait
        int pos = row_pos[row];
        int page = k_cache != nullptr
                       ? block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE] : 0;
        bool normed = live && !is_v && q_w != nullptr;
        bool rotate = live && !is_v && rot_half == half;
        float4 co = make_float4(1.0f, 1.0f, 1.0f, 1.0f), si = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float4 wl = co, wh = co;
        if (rotate) {
            co = load4(cs + (size_t)pos * half + at4);
            si = load4(sn + (size_t)pos * half + at4);
        }
        if (normed) {
            const TW *w = is_q ? q_w : k_w;
            wl = load4(w + at4);
            wh = load4(w + half + at4);
        }
        if (!waited) {
            pdl_wait();
            waited = true;
        }

        float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
        if (live) {
            const float *src = qkv + (size_t)row * slots * hd + (size_t)hs * hd + at4;
            for (int s0 = 0; s0 < S; s0 += 4) {
                float4 a[4], b[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (s0 + u < S) {
                        a[u] = load4(src + (size_t)(s0 + u) * split_stride);
                        b[u] = load4(src + (size_t)(s0 + u) * split_stride + half);
                    }
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (s0 + u < S) {
                        lo.x += a[u].x; lo.y += a[u].y; lo.z += a[u].z; lo.w += a[u].w;
                        hi.x += b[u].x; hi.y += b[u].y; hi.z += b[u].z; hi.w += b[u].w;
                    }
            }
        }
        float ss = lo.x * lo.x;
        ss = fmaf(lo.y, lo.y, ss); ss = fmaf(lo.z, lo.z, ss); ss = fmaf(lo.w, lo.w, ss);
        ss = fmaf(hi.x, hi.x, ss); ss = fmaf(hi.y, hi.y, ss);
        ss = fmaf(hi.z, hi.z, ss); ss = fmaf(hi.w, hi.w, ss);
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1)
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (!live)
            continue;
        TC *dst;
        if (is_q) {
            dst = q_out + ((size_t)row * nh + hs) * hd;
        } else {
            if (k_cache == nullptr)
                continue;
            int kvh = !is_v ? hs - nh : hs - nh - nkv;
            size_t at = (((size_t)page * nkv + kvh) * PAGE + (pos % PAGE)) * hd;
            dst = (!is_v ? k_cache : v_cache) + at;
        }
        if (normed) {
            float scale = 1.0f / sqrtf(ss / (float)hd + eps);
            lo.x = (lo.x * scale) * wl.x; lo.y = (lo.y * scale) * wl.y;
            lo.z = (lo.z * scale) * wl.z; lo.w = (lo.w * scale) * wl.w;
            hi.x = (hi.x * scale) * wh.x; hi.y = (hi.y * scale) * wh.y;
            hi.z = (hi.z * scale) * wh.z; hi.w = (hi.w * scale) * wh.w;
        }
        if (rotate) {
            float4 a = lo, b = hi;
            lo = make_float4(a.x * co.x - b.x * si.x, a.y * co.y - b.y * si.y,
                             a.z * co.z - b.z * si.z, a.w * co.w - b.w * si.w);
            hi = make_float4(a.x * si.x + b.x * co.x, a.y * si.y + b.y * co.y,
                             a.z * si.z + b.z * co.z, a.w * si.w + b.w * co.w);
        }
        store4(dst + at4, lo);
        store4(dst + half + at4, hi);
    }
}

// The same arithmetic, head by head, for many rows: a block has one row, its four
// warps take the row's groups of head slots in turn, three groups at a time so that
// their loads are in flight together.  What belongs to the row (position, page,
// rotation, norm weights) is fetched once per warp instead of once per group; the
// kernel above spends three quarters of its instructions on that.  Each head's sums
// run in the order of the kernel above, so that which of the two runs changes nothing.
template <typename TC, typename TW, int LPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_row_kernel(
    const float *__restrict__ qkv, int S, size_t split_stride, const TW *__restrict__ q_w,
    const TW *__restrict__ k_w, float eps, const float *__restrict__ cs,
    const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table, int bt_stride,
    TC *__restrict__ q_out, TC *__restrict__ k_cache, TC *__restrict__ v_cache, int n, int nh,
    int nkv)
{
    constexpr int SLOTS_PER_WARP = 32 / LPH, U = 3;
    constexpr int half = 4 * LPH, hd = 2 * half;
    pdl_trigger();
    unsigned row = blockIdx.x;
    int slots = nh + 2 * nkv;
    int groups = (slots + SLOTS_PER_WARP - 1) / SLOTS_PER_WARP;
    int at4 = 4 * (threadIdx.x % LPH), sub = threadIdx.x / LPH;
    int pos = row_pos[row];
    int page = k_cache != nullptr ? block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE] : 0;
    bool has_norm = q_w != nullptr, has_rot = rot_half == half;
    float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    float4 co = one, si = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 qwl = one, qwh = one, kwl = one, kwh = one;
    if (has_rot) {
        co = load4(cs + (size_t)pos * half + at4);
        si = load4(sn + (size_t)pos * half + at4);
    }
    if (has_norm) {
        qwl = load4(q_w + at4);
        qwh = load4(q_w + half + at4);
        kwl = load4(k_w + at4);
        kwh = load4(k_w + half + at4);
    }
    pdl_wait();
    const float *src_row = qkv + (size_t)row * slots * hd + at4;
    TC *q_row = q_out + (size_t)row * nh * hd + at4;
    size_t cache_at = ((size_t)page * nkv * PAGE + (pos % PAGE)) * hd + at4;
    for (int g0 = threadIdx.y; g0 < groups; g0 += 4 * U) {
        float4 lo[U], hi[U];
        int hs[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            int g = g0 + 4 * u;
            hs[u] = g < groups && g * SLOTS_PER_WARP + sub < slots ? g * SLOTS_PER_WARP + sub : -1;
            lo[u] = hi[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        for (int s = 0; s < S; s++) {
            float4 a[U], b[U];
#pragma unroll
            for (int u = 0; u < U; u++)
                if (hs[u] >= 0) {
                    const float *src = src_row + (size_t)s * split_stride + (size_t)hs[u] * hd;
                    a[u] = load4(src);
                    b[u] = load4(src + half);
                }
#pragma unroll
            for (int u = 0; u < U; u++)
                if (hs[u] >= 0) {
                    lo[u].x += a[u].x; lo[u].y += a[u].y; lo[u].z += a[u].z; lo[u].w += a[u].w;
                    hi[u].x += b[u].x; hi[u].y += b[u].y; hi[u].z += b[u].z; hi[u].w += b[u].w;
                }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            float4 l = lo[u], h = hi[u];
            float ss = l.x * l.x;
            ss = fmaf(l.y, l.y, ss); ss = fmaf(l.z, l.z, ss); ss = fmaf(l.w, l.w, ss);
            ss = fmaf(h.x, h.x, ss); ss = fmaf(h.y, h.y, ss);
            ss = fmaf(h.z, h.z, ss); ss = fmaf(h.w, h.w, ss);
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1)
                ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (hs[u] < 0)
                continue;
            bool is_q = hs[u] < nh, is_v = hs[u] >= nh + nkv;
            TC *dst;
            if (is_q) {
                dst = q_row + (size_t)hs[u] * hd;
            } else {
                if (k_cache == nullptr)
                    continue;
                int kvh = !is_v ? hs[u] - nh : hs[u] - nh - nkv;
                dst = (!is_v ? k_cache : v_cache) + cache_at + (size_t)kvh * PAGE * hd;
            }
            if (!is_v && has_norm) {
                float scale = 1.0f / sqrtf(ss / (float)hd + eps);
                float4 wl = is_q ? qwl : kwl, wh = is_q ? qwh : kwh;
                l.x = (l.x * scale) * wl.x; l.y = (l.y * scale) * wl.y;
                l.z = (l.z * scale) * wl.z; l.w = (l.w * scale) * wl.w;
                h.x = (h.x * scale) * wh.x; h.y = (h.y * scale) * wh.y;
                h.z = (h.z * scale) * wh.z; h.w = (h.w * scale) * wh.w;
            }
            if (!is_v && has_rot) {
                float4 a = l, b = h;
                l = make_float4(a.x * co.x - b.x * si.x, a.y * co.y - b.y * si.y,
                                a.z * co.z - b.z * si.z, a.w * co.w - b.w * si.w);
                h = make_float4(a.x * si.x + b.x * co.x, a.y * si.y + b.y * co.y,
                                a.z * si.z + b.z * co.z, a.w * si.w + b.w * co.w);
            }
            store4(dst, l);
            store4(dst + half, h);
        }
    }
}

}  // namespace jb

using namespace jb;

extern "C" int jb_rope_table(float *cs, float *sn, const float *inv_freq, int n_pos, int half,
                             cudaStream_t st)
{
    size_t total = (size_t)n_pos * half;
    if (total == 0)
        return JB_OK;
    launch(rope_table_kernel, (unsigned)((total + 255) / 256), 256, 0, st, cs, sn, inv_freq, n_pos,
           half);
    return launch_status();
}

extern "C" int jb_qk_norm_rope_append(const float *qkv, int S, long long split_stride,
                                      const void *q_w, const void *k_w, int w_dt, float eps,
                                      const float *cs, const float *sn, int rot_half,
                                      const int32_t *row_pos, const int32_t *row_seq,
                                      const int32_t *block_table, int bt_stride, void *q_out,
                                      void *k_cache, void *v_cache, int cache_dt, int n, int nh,
                                      int nkv, int hd, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    // the whole head is rotated or nothing is; a head has at most 512 values
    if (hd % 2 || hd > 512 || (rot_half != hd / 2 && rot_half != 0))
        return JB_EINVAL;
    if ((q_w == nullptr) != (k_w == nullptr))
        return JB_EINVAL;
    int slots = nh + 2 * nkv;
    dim3 block(32, 4);
    auto aligned = [](const void *p, size_t to) { return (uintptr_t)p % to == 0; };
    size_t w_to = w_dt == JB_F32 ? 16 : 8, c_to = cache_dt == JB_F32 ? 16 : 8;
    bool vec = (hd == 32 || hd == 64 || hd == 128 || hd == 256) && split_stride % 4 == 0 &&
               aligned(qkv, 16) && aligned(cs, 16) && aligned(sn, 16) && aligned(q_w, w_to) &&
               aligned(k_w, w_to) && aligned(q_out, c_to) && aligned(k_cache, c_to) &&
               aligned(v_cache, c_to);
    if (vec) {
        int per_warp = 32 / (hd / 8);
        size_t tasks = (size_t)n * ((slots + per_warp - 1) / per_warp);
        if (tasks > 0xffffffffu)
            return JB_EINVAL;
        unsigned grid = (unsigned)std::min<size_t>((tasks + 3) / 4, (size_t)sm_count() * 16);
        // from 256 rows on a block per row: fewer instructions; below, more warps per row
        bool by_row = n >= 256;
#define JB_ROPE_V(TC, TW, L)                                                                   \
    do {                                                                                       \
        if (by_row)                                                                            \
            launch(qk_norm_rope_append_row_kernel<TC, TW, L>, (unsigned)n, block, 0, st,       \
                qkv, S, (size_t)split_stride, (const TW *)q_w, (const TW *)k_w, eps, cs, sn,   \
                rot_half, row_pos, row_seq, block_table, bt_stride, (TC *)q_out,               \
                (TC *)k_cache, (TC *)v_cache, n, nh, nkv);                                     \
        else                                                                                   \
            launch(qk_norm_rope_append_vec_kernel<TC, TW, L>, grid, block, 0, st,              \
                qkv, S, (size_t)split_stride, (const TW *)q_w, (const TW *)k_w, eps, cs, sn,   \
                rot_half, row_pos, row_seq, block_table, bt_stride, (TC *)q_out,               \
                (TC *)k_cache, (TC *)v_cache, n, nh, nkv);                                     \
    } while (0)
#define JB_ROPE_VL(TC, TW)                                                                     \
    do {                                                                                       \
        if (hd == 32)                                                                          \
            JB_ROPE_V(TC, TW, 4);                                                              \
        else if (hd == 64)                                                                     \
            JB_ROPE_V(TC, TW, 8);                                                              \
        else if (hd == 128)                                                                    \
            JB_ROPE_V(TC, TW, 16);                                                             \
        else                                                                                   \
            JB_ROPE_V(TC, TW, 32);                                                             \
    } while (0)
        if (cache_dt == JB_F32 && w_dt == JB_F32)
            JB_ROPE_VL(float, float);
        else if (cache_dt == JB_F32 && w_dt == JB_BF16)
            JB_ROPE_VL(float, bf16);
        else if (cache_dt == JB_BF16 && w_dt == JB_F32)
            JB_ROPE_VL(bf16, float);
        else if (cache_dt == JB_BF16 && w_dt == JB_BF16)
            JB_ROPE_VL(bf16, bf16);
        else
            return JB_EINVAL;
#undef JB_ROPE_V
#undef JB_ROPE_VL
        return launch_status();
    }
    size_t tasks = (size_t)n * slots;
    if (tasks > 0xffffffffu)
        return JB_EINVAL;
    unsigned grid = (unsigned)((tasks + 3) / 4);
    int pairs = (hd / 2 + 31) / 32;
#define JB_ROPE_P(TC, TW, P)                                                                   \
    launch(qk_norm_rope_append_kernel<TC, TW, P>, grid, block, 0, st,                          \
        qkv, S, (size_t)split_stride, (const TW *)q_w, (const TW *)k_w, eps, cs, sn, rot_half, \
        row_pos, row_seq, block_table, bt_stride, (TC *)q_out, (TC *)k_cache, (TC *)v_cache, n, \
        nh, nkv, hd)
#define JB_ROPE(TC, TW)                                                                        \
    do {                                                                                       \
        if (pairs <= 1)                                                                        \
            JB_ROPE_P(TC, TW, 1);                                                              \
        else if (pairs <= 2)                                                                   \
            JB_ROPE_P(TC, TW, 2);                                                              \
        else if (pairs <= 4)                                                                   \
            JB_ROPE_P(TC, TW, 4);                                                              \
        else                                                                                   \
            JB_ROPE_P(TC, TW, 8);                                                              \
    } while (0)
    if (cache_dt == JB_F32 && w_dt == JB_F32)
        JB_ROPE(float, float);
    else if (cache_dt == JB_F32 && w_dt == JB_BF16)
        JB_ROPE(float, bf16);
    else if (cache_dt == JB_BF16 && w_dt == JB_F32)
        JB_ROPE(bf16, float);
    else if (cache_dt == JB_BF16 && w_dt == JB_BF16)
        JB_ROPE(bf16, bf16);
    else
        return JB_EINVAL;
#undef JB_ROPE_P
#undef JB_ROPE
    return launch_status();
}
