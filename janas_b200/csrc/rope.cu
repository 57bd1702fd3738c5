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

// One warp per (row, run of HPW head slots); head slots are the q heads, then
// the k heads, then the v heads of the row's fused [q | k | v] vector.  PAIRS is
// how many (low, high) pairs of a head a lane holds: ceil(hd / 64).  With many
// rows a warp takes several head slots of its row in turn, so that the row's
// rotation table and the norm weights are fetched once for all of them.
//
// qkv: S stacked [n, (nh + 2 nkv) hd] float partial sums.
// q_out: [n, nh, hd] in the cache's type.  K and V go to page
// block_table[seq][pos / PAGE] of k_cache / v_cache, which are laid out
// [page][kv head][PAGE][hd].
template <typename TC, typename TW, int PAIRS, int HPW>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_kernel(
    const float *__restrict__ qkv, int S, size_t split_stride, const TW *__restrict__ q_w,
    const TW *__restrict__ k_w, float eps, const float *__restrict__ cs,
    const float *__restrict__ sn, int rot_half, const int32_t *__restrict__ row_pos,
    const int32_t *__restrict__ row_seq, const int32_t *__restrict__ block_table, int bt_stride,
    TC *__restrict__ q_out, TC *__restrict__ k_cache, TC *__restrict__ v_cache, int n, int nh,
    int nkv, int hd)
{
    constexpr int hpw = HPW;
    pdl_trigger();
    unsigned slots = nh + 2 * nkv;
    unsigned runs = (slots + hpw - 1) / hpw;          // runs of head slots per row
    unsigned task = blockIdx.x * blockDim.y + threadIdx.y;
    if (task >= (unsigned)n * runs)
        return;
    unsigned row = task / runs, hs0 = (task - row * runs) * hpw;
    unsigned hs1 = min(hs0 + hpw, slots);
    int lane = threadIdx.x;
    int half = hd / 2;

    // Positions, page tables, rotation tables and norm weights were written long
    // before the kernel before this one: they are fetched before the wait.
    int pos = row_pos[row];
    int page = k_cache != nullptr
                   ? block_table[(size_t)row_seq[row] * bt_stride + pos / PAGE] : 0;
    bool rotate_any = rot_half == half;
    float co[PAIRS], si[PAIRS], wql[PAIRS], wqh[PAIRS], wkl[PAIRS], wkh[PAIRS];
#pragma unroll
    for (int j = 0; j < PAIRS; j++) {
        int i = lane + 32 * j;
        co[j] = 1.0f;
        si[j] = 0.0f;
        wql[j] = wqh[j] = wkl[j] = wkh[j] = 1.0f;
        if (i < half) {
            if (rotate_any) {
                co[j] = cs[(size_t)pos * rot_half + i];
                si[j] = sn[(size_t)pos * rot_half + i];
            }
            if (q_w != nullptr) {
                wql[j] = to_f(q_w[i]);
                wqh[j] = to_f(q_w[i + half]);
                wkl[j] = to_f(k_w[i]);
                wkh[j] = to_f(k_w[i + half]);
            }
        }
    }
    pdl_wait();

    // every head of this warp is fetched before the first is worked on
    float lo[HPW][PAIRS], hi[HPW][PAIRS];
#pragma unroll
    for (int k = 0; k < HPW; k++) {
        unsigned hs = hs0 + k;
        const float *src = qkv + (size_t)row * slots * hd + (size_t)hs * hd;
#pragma unroll
        for (int j = 0; j < PAIRS; j++) {
            int i = lane + 32 * j;
            lo[k][j] = hi[k][j] = 0.0f;
            if (hs < hs1 && i < half) {
                lo[k][j] = add_partials(0.0f, src + i, S, split_stride);
                hi[k][j] = add_partials(0.0f, src + i + half, S, split_stride);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < HPW; k++) {
        unsigned hs = hs0 + k;
        if (hs >= hs1)
            break;
        bool is_q = hs < (unsigned)nh;
        bool is_v = hs >= (unsigned)(nh + nkv);
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
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < PAIRS; j++) {
            ss = fmaf(lo[k][j], lo[k][j], ss);
            ss = fmaf(hi[k][j], hi[k][j], ss);
        }
        bool normed = !is_v && q_w != nullptr;
        float scale = 1.0f;
        if (normed) {
            ss = warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)hd + eps);
        }
        bool rotate = !is_v && rotate_any;
#pragma unroll
        for (int j = 0; j < PAIRS; j++) {
            int i = lane + 32 * j;
            if (i < half) {
                float a = lo[k][j], b = hi[k][j];
                if (normed) {
                    a = (a * scale) * (is_q ? wql[j] : wkl[j]);
                    b = (b * scale) * (is_q ? wqh[j] : wkh[j]);
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
    // few rows: a warp per head slot, for the shortest chain; many rows: several
    // head slots per warp, for fewer fetches of what the row's heads share
    int slots = nh + 2 * nkv;
    int hpw = n >= 256 && slots >= 8 ? 4 : 1;
    size_t tasks = (size_t)n * ((slots + hpw - 1) / hpw);
    if (tasks > 0xffffffffu)
        return JB_EINVAL;
    dim3 block(32, 4);
    unsigned grid = (unsigned)((tasks + 3) / 4);
    int pairs = (hd / 2 + 31) / 32;
#define JB_ROPE_PH(TC, TW, P, H)                                                               \
    launch(qk_norm_rope_append_kernel<TC, TW, P, H>, grid, block, 0, st,                       \
        qkv, S, (size_t)split_stride, (const TW *)q_w, (const TW *)k_w, eps, cs, sn, rot_half, \
        row_pos, row_seq, block_table, bt_stride, (TC *)q_out, (TC *)k_cache, (TC *)v_cache, n, \
        nh, nkv, hd)
#define JB_ROPE_P(TC, TW, P)                                                                   \
    do {                                                                                       \
        if (hpw == 1)                                                                          \
            JB_ROPE_PH(TC, TW, P, 1);                                                          \
        else                                                                                   \
            JB_ROPE_PH(TC, TW, P, 4);                                                          \
    } while (0)
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
#undef JB_ROPE_PH
#undef JB_ROPE
    return launch_status();
}
