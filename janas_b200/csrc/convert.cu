// Element type conversions on the device: bfloat16 <-> float32 (0: float32,
// 1: bfloat16, as everywhere in the kernels' C interface).  Used when weights of
// different stored types are fused into one matrix.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace {

template <typename S, typename D>
__global__ void convert_kernel(const S *__restrict__ src, D *__restrict__ dst, long long n)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += step) {
        float v;
        if constexpr (sizeof(S) == 4)
            v = src[i];
        else
            v = __bfloat162float(src[i]);
        if constexpr (sizeof(D) == 4)
            dst[i] = v;
        else
            dst[i] = __float2bfloat16_rn(v);
    }
}

}  // namespace

extern "C" int jb_convert(const void *src, int src_dt, void *dst, int dst_dt, long long n,
                          cudaStream_t st)
{
    if (n <= 0)
        return 0;
    if ((src_dt != 0 && src_dt != 1) || (dst_dt != 0 && dst_dt != 1))
        return -1;
    long long b = (n + 255) / 256;
    unsigned blocks = (unsigned)(b > 148 * 16 ? 148 * 16 : b);
    if (src_dt == dst_dt) {
        size_t bytes = (size_t)n * (src_dt == 0 ? 4 : 2);
        return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st) == cudaSuccess ? 0 : -2;
    }
    if (src_dt == 1)
        convert_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16 *)src, (float *)dst, n);
    else
        convert_kernel<<<blocks, 256, 0, st>>>((const float *)src, (__nv_bfloat16 *)dst, n);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
