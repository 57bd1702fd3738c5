// Normal random numbers written straight into device memory: the random-weights
// mode for models too large to draw on the host (a Qwen3-32B-size model is
// 65 GB).  Counter-based: value i of a tensor depends on the tensor's seed and on
// i alone (splitmix64 of seed + i gives two uniforms, Box-Muller turns them into
// one normal), so the grid's shape does not matter.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ unsigned long long mix(unsigned long long z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T *out, long long n, unsigned long long seed, float mean, float sd)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long step = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += step) {
        unsigned long long r = mix(seed + (unsigned long long)i * 0xD1342543DE82EF95ull);
        // two uniforms in (0, 1]
        float u1 = ((float)(unsigned)(r >> 40) + 1.0f) * (1.0f / 16777216.0f);
        float u2 = (float)(unsigned)((r >> 8) & 0xffffff) * (1.0f / 16777216.0f);
        float v = mean + sd * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        if constexpr (sizeof(T) == 4)
            out[i] = v;
        else
            out[i] = __float2bfloat16_rn(v);
    }
}

}  // namespace

extern "C" int jb_fill_normal(void *out, int dt, long long n, unsigned long long seed, float mean,
                              float sd, cudaStream_t st)
{
    if (n <= 0)
        return 0;
    if (dt != 0 && dt != 1)
        return -1;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16)
        blocks = 148 * 16;
    if (dt == 0)
        fill_normal_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((float *)out, n, seed, mean, sd);
    else
        fill_normal_kernel<__nv_bfloat16>
            <<<(unsigned)blocks, 256, 0, st>>>((__nv_bfloat16 *)out, n, seed, mean, sd);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
