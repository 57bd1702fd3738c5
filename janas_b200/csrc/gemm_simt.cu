// out[n, m] = A[n, k] . W[m, k]^T with plain float multiply-adds.
//
// This is the matrix product of the true 32-bit path and the fallback for
// shapes and type mixes the tensor-core kernel refuses.  Every output value is
// computed by one fixed recipe, whatever n is and wherever the row lies in the
// batch, so a row's result is the same bits however the tokens are cut into
// steps: k is cut into segments of SEG values at fixed places; within a segment
// the products are added by one chain of fmaf in ascending order from zero; the
// segments' sums are added in ascending order.  Two kernels follow the recipe:
// one for many tokens (a thread walks all segments of its outputs) and one for
// the few tokens of a decode step (a block per segment, so that a narrow matrix
// still keeps every SM's loads in flight; the segments' sums go through scratch
// and a second kernel adds them in order).  A and W are float or bfloat16
// (widened exactly); no reduced-precision matrix mode is involved.
//
// The reference computes y = W x with rows of W as output features
// (src/llm/model_load.c:452, src/llm/model_attn.c:234-255); its products are
// over quantized blocks and are not reproduced.
#include "common.cuh"
#include "kernels.h"

namespace jb {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int SEG = 512;      // k per segment; a multiple of BK and of SK_K

template <typename T>
__device__ __forceinline__ void load4(const T *base, size_t row, int rows, int col, int k,
                                      bool vec, float *v)
{
    v[0] = v[1] = v[2] = v[3] = 0.0f;
    if ((int)row >= rows)
        return;
    const T *p = base + row * (size_t)k + col;
    if (vec && col + 3 < k) {
        if constexpr (sizeof(T) == 4) {
            float4 f = *reinterpret_cast<const float4 *>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            uint2 u = *reinterpret_cast<const uint2 *>(p);
            v[0] = __uint_as_float(u.x << 16);
            v[1] = __uint_as_float(u.x & 0xffff0000u);
            v[2] = __uint_as_float(u.y << 16);
            v[3] = __uint_as_float(u.y & 0xffff0000u);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (col + i < k)
            v[i] = to_f(p[i]);
}

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA *__restrict__ A, const TW *__restrict__ W, float *__restrict__ out,
                 int n, int m, int k, bool vec)
{
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    pdl_trigger();
    pdl_wait();
    int tid = threadIdx.x;
    int tx = tid % 16, ty = tid / 16;
    size_t n0 = (size_t)blockIdx.y * BM, m0 = (size_t)blockIdx.x * BN;
    int lr = tid / 4, lc = (tid % 4) * 4;  // this thread's 4 values of a 64 x 16 tile

    float acc[4][4], total[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = total[i][j] = 0.0f;

    // the next tile's values are on their way while this tile is multiplied
    float a4[4], w4[4];
    load4<TA>(A, n0 + lr, n, lc, k, vec, a4);
    load4<TW>(W, m0 + lr, m, lc, k, vec, w4);
    for (int k0 = 0; k0 < k; k0 += BK) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lc + i][lr] = a4[i];
            Ws[lc + i][lr] = w4[i];
        }
        __syncthreads();
        if (k0 + BK < k) {
            load4<TA>(A, n0 + lr, n, k0 + BK + lc, k, vec, a4);
            load4<TW>(W, m0 + lr, m, k0 + BK + lc, k, vec, w4);
        }
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a[i] = As[kk][ty * 4 + i];
                w[i] = Ws[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        if ((k0 + BK) % SEG == 0 || k0 + BK >= k) {
            // a segment ends: its sum joins the total; the first one is the total
            bool first = k0 < SEG;
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    total[i][j] = first ? acc[i][j] : total[i][j] + acc[i][j];
                    acc[i][j] = 0.0f;
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        size_t r = n0 + ty * 4 + i;
        if (r >= (size_t)n)
            continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            size_t c = m0 + tx * 4 + j;
            if (c < (size_t)m)
                out[r * m + c] = total[i][j];
        }
    }
}

// The same recipe for up to 16 tokens (a decode step): a block takes 128 features,
// all tokens and ONE segment of k, and writes the segment's sums to `part`
// [segments, n, m]; a thread owns four features and four tokens (16 chains of
// fmaf), so that a value read from shared memory feeds four multiply-adds.  With one
// segment in all, the sums are the result and go to `out` directly.
constexpr int SK_FEATS = 128, SK_K = 32, SK_THREADS = 128, SK_MAX_N = 16;
static_assert(SEG % BK == 0 && SEG % SK_K == 0, "segments end where both kernels' tiles end");

template <typename TA, typename TW>
__global__ void __launch_bounds__(SK_THREADS)
gemm_simt_skinny_kernel(const TA *__restrict__ A, const TW *__restrict__ W, float *__restrict__ part,
                        int n, int m, int k, bool vec)
{
    __shared__ __align__(16) float Ws[SK_K][SK_FEATS + 4];
    __shared__ __align__(16) float As[SK_K][SK_MAX_N + 4];
    pdl_trigger();
    pdl_wait();
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int fx = lane, g = warp;                             // features 4 fx .. 4 fx + 3, tokens 4 g .. 4 g + 3
    size_t m0 = (size_t)blockIdx.x * SK_FEATS;
    int ka = blockIdx.y * SEG, kb = min(k, ka + SEG);    // this block's segment
    // loads of a 128 x 32 weight tile: rows lane + 32 j, the warp's quarter of k;
    // of the 16 x 32 token tile: row tid % 16, four values of k
    int wk = warp * 8, ar = tid & 15, ak = (tid >> 4) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = 0.0f;
    float w4[4][2][4], a4[4];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int h = 0; h < 2; h++)
                load4<TW>(W, m0 + lane + 32 * j, m, k0 + wk + 4 * h, k, vec, w4[j][h]);
        load4<TA>(A, (size_t)ar, n, k0 + ak, k, vec, a4);
    };
    fetch(ka);
    for (int k0 = ka; k0 < kb; k0 += SK_K) {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    Ws[wk + 4 * h + i][lane + 32 * j] = w4[j][h][i];
#pragma unroll
        for (int i = 0; i < 4; i++)
            As[ak + i][ar] = a4[i];
        __syncthreads();
        if (k0 + SK_K < kb)
            fetch(k0 + SK_K);
#pragma unroll
        for (int kk = 0; kk < SK_K; kk++) {
            float4 w = *reinterpret_cast<const float4 *>(&Ws[kk][4 * fx]);
            float4 a = *reinterpret_cast<const float4 *>(&As[kk][4 * g]);
            float wv[4] = {w.x, w.y, w.z, w.w}, av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    acc[i][j] = fmaf(av[j], wv[i], acc[i][j]);
        }
    }
    float *dst = part + (size_t)blockIdx.y * n * m;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int r = 4 * g + j;
        if (r >= n)
            continue;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            size_t c = m0 + 4 * fx + i;
            if (c < (size_t)m)
                dst[(size_t)r * m + c] = acc[i][j];
        }
    }
}

// out = ((part[0] + part[1]) + part[2]) + ...: the segments' sums in ascending order.
__global__ void __launch_bounds__(256)
gemm_simt_join_kernel(const float *__restrict__ part, float *__restrict__ out, long long count,
                      int segments)
{
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count)
        return;
    float t = part[i];
    for (int s = 1; s < segments; s++)
        t = t + part[(size_t)s * count + i];
    out[i] = t;
}

}  // namespace jb

using namespace jb;

// Floats of scratch that jb_gemm_simt wants for this shape (0: none).
extern "C" long long jb_gemm_simt_scratch(int n, int m, int k)
{
    int segments = (k + SEG - 1) / SEG;
    if (n <= 0 || n > SK_MAX_N || segments <= 1)
        return 0;
    return (long long)segments * n * m;
}

// scratch: jb_gemm_simt_scratch(n, m, k) floats (may be null when that is 0).
extern "C" int jb_gemm_simt(const void *A, int a_dt, const void *W, int w_dt, float *out, int n,
                            int m, int k, float *scratch, cudaStream_t st)
{
    if (n <= 0 || m <= 0)
        return JB_OK;
    if (k <= 0)
        return JB_EINVAL;
    dim3 grid((m + BN - 1) / BN, (n + BM - 1) / BM);
    if (grid.y > 65535)
        return JB_EINVAL;
    bool vec = k % 4 == 0 && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
    bool skinny = n <= SK_MAX_N;
    int segments = (k + SEG - 1) / SEG;
    if (skinny && segments > 1 && scratch == nullptr)
        return JB_EINVAL;
    dim3 sgrid((m + SK_FEATS - 1) / SK_FEATS, segments);
    float *part = segments > 1 ? scratch : out;
#define JB_GEMM(TA, TW)                                                                       \
    if (skinny)                                                                               \
        launch(gemm_simt_skinny_kernel<TA, TW>, sgrid, SK_THREADS, 0, st, (const TA *)A,      \
               (const TW *)W, part, n, m, k, vec);                                            \
    else                                                                                      \
        launch(gemm_simt_kernel<TA, TW>, grid, 256, 0, st, (const TA *)A, (const TW *)W, out, n, m, k, vec)
    if (a_dt == JB_F32 && w_dt == JB_F32) {
        JB_GEMM(float, float);
    } else if (a_dt == JB_F32 && w_dt == JB_BF16) {
        JB_GEMM(float, bf16);
    } else if (a_dt == JB_BF16 && w_dt == JB_F32) {
        JB_GEMM(bf16, float);
    } else if (a_dt == JB_BF16 && w_dt == JB_BF16) {
        JB_GEMM(bf16, bf16);
    } else {
        return JB_EINVAL;
    }
#undef JB_GEMM
    if (skinny && segments > 1) {
        if (cudaGetLastError() != cudaSuccess)
            return JB_ELAUNCH;
        long long count = (long long)n * m;
        launch(gemm_simt_join_kernel, (unsigned)((count + 255) / 256), 256, 0, st, (const float *)part,
               out, count, segments);
    }
    return launch_status();
}
