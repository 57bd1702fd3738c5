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

// One warp per (row, head slot); head slots are the q heads, then the k
// heads, then the v heads of the row's fused [q | k | v] vector.
//
// qkv: S stacked [n, (nh + 2 nkv) hd] float partial sums.
// q_out: [n, nh, hd] in the cache's type.  K and V go to page
// block_table[seq][pos / PAGE] of k_cache / v_cache, which are laid out
// [page][kv head][PAGE][hd].
template <typename TC, typename TW>
__global__ void qk_norm_rope_append_kernel(
    const float *__restrict__ qkv, int S, size_t split_stride, const TW *__restrict__ q_w,
    const TW *__restrict__ k_w, float eps, const float *__restrict__ cs,
    const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table, int bt_stride,
    TC *__restrict__ q_out, TC *__restrict__ k_cache, TC *__restrict__ v_cache, int n, int nh,
    int nkv, int hd, int table_half)
{
    pdl_trigger();
    pdl_wait();
    int slots = nh + 2 * nkv;
    size_t task = (size_t)blockIdx.x * blockDim.y + threadIdx.y;
    if (task >= (size_t)n * slots)
        return;
    int row = (int)(task / slots), hs = (int)(task % slots);
    int lane = threadIdx.x;
    int pos = row_pos[row];
    size_t width = (size_t)slots * hd;
    const float *src = qkv + (size_t)row * width + (size_t)hs * hd;

    TC *dst;
    if (hs < nh) {
        dst = q_out + ((size_t)row * nh + hs) * hd;
    } else {
        if (k_cache == nullptr)
            return;
        int kvh = hs < nh + nkv ? hs - nh : hs - nh - nkv;
        int page = block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE];
        size_t at = (((size_t)page * nkv + kvh) * PAGE + (pos % PAGE)) * hd;
        dst = (hs < nh + nkv ? k_cache : v_cache) + at;
    }

    if (hs >= nh + nkv) {  // V: the sum of the partial sums, as it is
        for (int i = lane; i < hd; i += 32) {
            dst[i] = from_f<TC>(add_partials(0.0f, src + i, S, split_stride));
        }
        return;
    }

    const TW *w = hs < nh ? q_w : k_w;
    // a head of up to 512 values: 16 per lane, held as 8 (low, high) pairs
    constexpr int MAXP = 8;
    int half = hd / 2;
    float lo[MAXP], hi[MAXP];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < MAXP; j++) {
        int i = lane + 32 * j;
        lo[j] = hi[j] = 0.0f;
        if (i < half) {
            lo[j] = add_partials(0.0f, src + i, S, split_stride);
            hi[j] = add_partials(0.0f, src + i + half, S, split_stride);
            ss = fmaf(lo[j], lo[j], ss);
            ss = fmaf(hi[j], hi[j], ss);
        }
    }
    float scale = 1.0f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    const float *c = cs + (size_t)pos * table_half;
    const float *sgn = sn + (size_t)pos * table_half;
#pragma unroll
    for (int j = 0; j < MAXP; j++) {
        int i = lane + 32 * j;
        if (i < half) {
            float a = lo[j], b = hi[j];
            if (w != nullptr) {
                a = (a * scale) * to_f(w[i]);
                b = (b * scale) * to_f(w[i + half]);
            }
            // the rotation covers the first 2 rot_half values of the head as
            // pairs (i, i + rot_half); with the whole head rotated that is
            // (i, i + half)
            if (rot_half == half) {
                float co = c[i], si = sgn[i];
                dst[i] = from_f<TC>(a * co - b * si);
                dst[i + half] = from_f<TC>(a * si + b * co);
            } else {
                dst[i] = from_f<TC>(a);
                dst[i + half] = from_f<TC>(b);
            }
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
    size_t tasks = (size_t)n * (nh + 2 * nkv);
    dim3 block(32, 4);
    unsigned grid = (unsigned)((tasks + 3) / 4);
    int table_half = rot_half;
#define JB_ROPE(TC, TW)                                                                        \
    launch(qk_norm_rope_append_kernel<TC, TW>, grid, block, 0, st,                             \
        qkv, S, (size_t)split_stride, (const TW *)q_w, (const TW *)k_w, eps, cs, sn, rot_half, \
        row_pos, row_seq, block_table, bt_stride, (TC *)q_out, (TC *)k_cache, (TC *)v_cache, n, \
        nh, nkv, hd, table_half)
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
#undef JB_ROPE
    return launch_status();
}
