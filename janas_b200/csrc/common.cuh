// Shared device helpers of the janas_b200 kernels (sm_100a).
//
// Storage types are float or __nv_bfloat16; all arithmetic is done in float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace jb {

typedef __nv_bfloat16 bf16;

// Positions a page of the cache holds.  The host side (cache/pages.py) uses the
// same number.
constexpr int PAGE = 64;

// Error codes returned by the launchers (0 = launched).
enum : int {
    JB_OK = 0,
    JB_EINVAL = -1,   // an argument the kernel does not take
    JB_ELAUNCH = -2,  // the launch itself failed (cudaGetLastError)
};

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// Four consecutive values at a 16-byte (float) or 8-byte (bfloat16) boundary.
template <typename T> __device__ __forceinline__ float4 load4(const T *p);
template <> __device__ __forceinline__ float4 load4<float>(const float *p)
{
    return *reinterpret_cast<const float4 *>(p);
}
template <> __device__ __forceinline__ float4 load4<bf16>(const bf16 *p)
{
    uint2 u = *reinterpret_cast<const uint2 *>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
template <typename T> __device__ __forceinline__ void store4(T *p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float *p, float4 v)
{
    *reinterpret_cast<float4 *>(p) = v;
}
template <> __device__ __forceinline__ void store4<bf16>(bf16 *p, float4 v)
{
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) =
        make_uint2(*reinterpret_cast<uint32_t *>(&a), *reinterpret_cast<uint32_t *>(&b));
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions depends only on the block size.  red: 32 floats of
// shared memory.
__device__ __forceinline__ float block_sum(float v, float *red)
{
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // red may still be read from an earlier call
    if (lane == 0)
        red[warp] = v;
    __syncthreads();
    float t = lane < nwarp ? red[lane] : 0.0f;
    return warp_sum(t);
}

// p[0] + p[stride] + ... + p[(S - 1) stride], added in that order to `v`.  Up
// to sixteen terms are fetched together, so the chain of additions does not also
// become a chain of memory latencies.
__device__ __forceinline__ float add_partials(float v, const float *__restrict__ p, int S,
                                              size_t stride)
{
    if (S == 1)
        return v + p[0];
    for (int s0 = 0; s0 < S; s0 += 16) {
        float t[16];
#pragma unroll
        for (int u = 0; u < 16; u++)
            t[u] = s0 + u < S ? p[(size_t)(s0 + u) * stride] : 0.0f;
#pragma unroll
        for (int u = 0; u < 16; u++)
            if (s0 + u < S)
                v += t[u];
    }
    return v;
}

// Programmatic dependent launch.  Every kernel of this library is launched with
// the attribute that lets its CTAs start while the kernel before it in the
// stream is still running.  pdl_trigger() (early in a kernel) allows the next
// kernel's CTAs to be scheduled once all of this kernel's CTAs have started;
// pdl_wait() blocks until the kernel before this one has completed and its
// writes are visible.  What a kernel does before pdl_wait() must not touch
// anything an earlier kernel writes or reads-and-frees: only its own shared and
// tensor memory and the (immutable) weights.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_x` along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t st, unsigned cluster_x, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Thread-block clusters: this CTA's rank, the two halves of the cluster-wide
// barrier, and a float read from the same shared-memory variable of another CTA.
__device__ __forceinline__ uint32_t cluster_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float cluster_read(const float *mine, uint32_t rank)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(mine), ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}

// A float written to the same shared-memory variable of another CTA of the cluster
// (seen there after the cluster-wide barrier).
__device__ __forceinline__ void cluster_write(float *mine, uint32_t rank, float v)
{
    uint32_t a = (uint32_t)__cvta_generic_to_shared(mine), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

// SMs of the current device (148 on a B200), asked once per device.
inline int sm_count()
{
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    int slot = dev >= 0 && dev < 64 ? dev : 0;
    if (sms[slot] == 0) {
        int n = 0;
        sms[slot] = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
                            n > 0 ? n : 148;
    }
    return sms[slot];
}

// Lets a kernel use `bytes` of dynamic shared memory on the current device; `done`
// is the caller's record (a bit per device) of where that has been said already.
template <typename Kernel>
inline bool allow_dynamic_smem(Kernel kern, int bytes, unsigned long long &done)
{
    int dev = 0;
    cudaGetDevice(&dev);
    bool tracked = dev >= 0 && dev < 64;
    if (tracked && (done >> dev & 1))
        return true;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
        cudaSuccess)
        return false;
    if (tracked)
        done |= 1ull << dev;
    return true;
}

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? JB_OK : JB_ELAUNCH;
}

}  // namespace jb
