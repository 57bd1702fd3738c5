// out[n, m] = A[n, k] . W[m, k]^T with plain float multiply-adds.
//
// This is the matrix product of the true 32-bit path and the fallback for
// shapes and type mixes the tensor-core kernel refuses.  Every output value is
// one thread's sum over k in ascending order, whatever n is and wherever the
// row lies in the batch, so a row's result is the same bits however the tokens
// are cut into steps.  A and W are float or bfloat16 (widened exactly); no
// reduced-precision matrix mode is involved.
//
// The reference computes y = W x with rows of W as output features
// (src/llm/model_load.c:452, src/llm/model_attn.c:234-255); its products are
// over quantized blocks and are not reproduced.
#include "common.cuh"
#include "kernels.h"

namespace jb {

constexpr int BM = 64, BN = 64, BK = 16;

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

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < k; k0 += BK) {
        float a4[4], w4[4];
        load4<TA>(A, n0 + lr, n, k0 + lc, k, vec, a4);
        load4<TW>(W, m0 + lr, m, k0 + lc, k, vec, w4);
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            As[lc + i][lr] = a4[i];
            Ws[lc + i][lr] = w4[i];
        }
        __syncthreads();
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
                out[r * m + c] = acc[i][j];
        }
    }
}

}  // namespace jb

using namespace jb;

extern "C" int jb_gemm_simt(const void *A, int a_dt, const void *W, int w_dt, float *out, int n,
                            int m, int k, cudaStream_t st)
{
    if (n <= 0 || m <= 0)
        return JB_OK;
    if (k <= 0)
        return JB_EINVAL;
    dim3 grid((m + BN - 1) / BN, (n + BM - 1) / BM);
    if (grid.y > 65535)
        return JB_EINVAL;
    bool vec = k % 4 == 0 && ((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0);
#define JB_GEMM(TA, TW)                                                                       \
    launch(gemm_simt_kernel<TA, TW>, grid, 256, 0, st, (const TA *)A, (const TW *)W, out, n, m, k, vec)
    if (a_dt == JB_F32 && w_dt == JB_F32)
        JB_GEMM(float, float);
    else if (a_dt == JB_F32 && w_dt == JB_BF16)
        JB_GEMM(float, bf16);
    else if (a_dt == JB_BF16 && w_dt == JB_F32)
        JB_GEMM(bf16, float);
    else if (a_dt == JB_BF16 && w_dt == JB_BF16)
        JB_GEMM(bf16, bf16);
    else
        return JB_EINVAL;
#undef JB_GEMM
    return launch_status();
}
