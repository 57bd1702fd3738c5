// Matrix products on the fifth-generation tensor cores (tcgen05), bfloat16 in,
// float accumulation in tensor memory, operands staged by TMA.
//
//     out[n, m] = A[n, k] . W[m, k]^T
//
// The weight matrix is the M operand of the instruction (128 output features per
// tile, one TMEM lane each) and the tokens are its N operand (16 to 256 per
// tile, one TMEM column each), so that a decode step with a handful of tokens
// still fills the 128-row instruction and a weight is read exactly once.  Both
// operands are K-major rows of 64 bfloat16 (128 bytes) in the 128-byte swizzle
// that TMA writes and the matrix descriptor names.
//
// A CTA computes one tile: 128 * MT features by BN tokens over one part of k
// (grid.z parts; each part writes its own float partial sum, added by whoever
// reads the product next, in a fixed order).  Warp 0 issues the TMA loads,
// warp 1 owns the tensor memory and issues the MMAs, warps 2..9 read the
// accumulator back (a thread per feature and half of the tokens) and store.  With EPI_SWIGLU the two
// weight tiles are the gate rows and the up rows of the same features and the
// epilogue writes SiLU(gate) * up in bfloat16.
//
// Every wait on an mbarrier has a time limit; when it runs out the CTA records
// it in an error word that the host reads (jb_gemm_tc_error), stops issuing
// work, waits once more (with the same limit) for the loads it has in flight,
// frees its tensor memory and returns.  No load uses cluster multicast.
//
// The reference has no counterpart: its products are quantized dot products on
// CPU threads or dp4a (src/llm/cuda/matvec.cu:344-414).
#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "kernels.h"
#include "tc_common.cuh"

namespace jb {

constexpr int BK = 64;              // k per stage: 128 bytes of bfloat16, one swizzle row
constexpr int TILE_M = 128;         // features per MMA
constexpr int W_TILE_BYTES = TILE_M * BK * 2;
constexpr int EPI_PARTIAL = 0;      // store float partial sums
constexpr int EPI_SWIGLU = 1;       // two tiles: gate and up; store SiLU(gate) * up as bfloat16
// one tile whose rows are 64 gate features and the 64 up features that pair with
// them: as many CTAs as the plain product has, for the few tokens of a decode step
constexpr int EPI_SWIGLU_HALF = 2;
constexpr int HALF_M = TILE_M / 2;
// warp 0 loads, warp 1 issues the MMAs, warps 2..9 read the accumulator back: a
// warp may read the 32 TMEM lanes of its index modulo 4, so two warps share each
// quarter of the features and take the 32-column groups in turn
constexpr int GEMM_THREADS = 320;

__device__ int g_gemm_tc_error;     // 0, or the code of the first wait that ran out

// The shared-memory matrix descriptor of a K-major tile of 128-byte rows in the
// 128-byte swizzle: start address, leading offset 1 (unused for this layout),
// 1024 bytes from one group of eight rows to the next, descriptor version 1,
// layout type 2 (128-byte swizzle); all offsets in units of 16 bytes.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// kind::f16 instruction descriptor: float accumulator (bits 4-5 = 1), bfloat16
// A and B (bits 7-9 and 10-12 = 1), both K-major, N / 8 at bit 17, M / 16 at 24.
__host__ __device__ constexpr uint32_t instr_desc(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(TILE_M >> 4) << 24);
}

// DEEP: a product whose CTAs are about as many as the SMs (the fused gate-up product
// of a decode step: 152 tiles) has one CTA on most SMs, so each keeps a stage more in
// flight; two of them still fit an SM, and one beside a CTA of the product after it.
template <int BN, int MT, bool DEEP = false> struct TileCfg {
    static constexpr int A_TILE_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = MT * W_TILE_BYTES + A_TILE_BYTES;
    // 2 CTAs per SM for the small tiles that stream weights, 1 for the large ones
    static constexpr int RING_BYTES = (BN <= 128 && MT == 1) ? (DEEP ? 110 : 100) * 1024 : 225 * 1024;
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES < 2 ? 2 : (RING_BYTES / STAGE_BYTES > 8 ? 8 : RING_BYTES / STAGE_BYTES);
    static constexpr int TMEM_COLS = MT * BN <= 32 ? 32 : MT * BN <= 64 ? 64 : MT * BN <= 128 ? 128 : MT * BN <= 256 ? 256 : 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment */ + 256 /* barriers */;
};

// The epilogues.  A thread owns one feature (a TMEM lane) and, with the other
// warp of its quarter, takes the groups of 32 token columns in turn (hgrp, hgrp
// + 2, ...); the read of the next group is in flight while the last one is stored.
//
// Float partial sums: tile t's tokens are columns [t BN, t BN + BN).
template <int BN, int MT>
__device__ __forceinline__ void store_partial(uint32_t taddr, int hgrp, float *__restrict__ dst,
                                              int f, int n0, int n, int m, int second_off)
{
    constexpr int COLS = MT * BN;
    if constexpr (BN < 32) {
        float v[16];
        if (hgrp != 0)
            return;
        tc_ld16(taddr, v);
        if (f < m) {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (n0 + j < n)
                    dst[(size_t)(n0 + j) * m + f] = v[j];
        }
    } else {
        uint32_t va[32], vb[32];
        auto store32 = [&](const uint32_t *v, int c) {
            int t = c / BN, c0 = c - t * BN;
            int ft = f + t * second_off;
            if (ft >= m)
                return;
            float *p = dst + (size_t)(n0 + c0) * m + ft;
            if (n0 + c0 + 32 <= n) {        // the usual case: no token is cut off
#pragma unroll
                for (int j = 0; j < 32; j++, p += m)
                    *p = __uint_as_float(v[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++, p += m)
                    if (n0 + c0 + j < n)
                        *p = __uint_as_float(v[j]);
            }
        };
        int c = 32 * hgrp;
        if (c < COLS) {
            tc_ld32_nowait(taddr + c, va);
#pragma unroll 1
            for (; c < COLS; c += 128) {
                tc_ld_wait();
                if (c + 64 < COLS)
                    tc_ld32_nowait(taddr + c + 64, vb);
                store32(va, c);
                if (c + 64 < COLS) {
                    tc_ld_wait();
                    if (c + 128 < COLS)
                        tc_ld32_nowait(taddr + c + 128, va);
                    store32(vb, c + 64);
                }
            }
        }
    }
}

// SiLU(gate) * up in bfloat16: the gate's tokens are columns [0, BN), the up
// projection's [BN, 2 BN).  SiLU(g) u = g u / (1 + 2^(-g log2 e)), with the
// approximate exponential and reciprocal (a few units in the last place of a
// float; the result is rounded to bfloat16).
template <int BN>
__device__ __forceinline__ void store_swiglu(uint32_t taddr, int hgrp, bf16 *__restrict__ out_act,
                                             int f, int ff, int n0, int n)
{
    uint32_t ga[32], ua[32], gb[32], ub[32];
    auto act32 = [&](const uint32_t *g, const uint32_t *u, int c0) {
        if (f >= ff)
            return;
        bf16 *p = out_act + (size_t)(n0 + c0) * ff + f;
        bool whole = n0 + c0 + 32 <= n;
#pragma unroll
        for (int j = 0; j < 32; j++, p += ff) {
            if (whole || n0 + c0 + j < n) {
                float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                float e = fast_exp2(gv * -1.4426950408889634f);
                *p = __float2bfloat16_rn(__fdividef(gv * uv, 1.0f + e));
            }
        }
    };
    int c = 32 * hgrp;
    if (c < BN) {
        tc_ld32_nowait(taddr + c, ga);
        tc_ld32_nowait(taddr + BN + c, ua);
#pragma unroll 1
        for (; c < BN; c += 128) {
            tc_ld_wait();
            if (c + 64 < BN) {
                tc_ld32_nowait(taddr + c + 64, gb);
                tc_ld32_nowait(taddr + BN + c + 64, ub);
            }
            act32(ga, ua, c);
            if (c + 64 < BN) {
                tc_ld_wait();
                if (c + 128 < BN) {
                    tc_ld32_nowait(taddr + c + 128, ga);
                    tc_ld32_nowait(taddr + BN + c + 128, ua);
                }
                act32(gb, ub, c + 64);
            }
        }
    }
}

// The same for a tile whose TMEM lanes [0, 64) are gate features and [64, 128) the
// up features of the same indices: the warps of the upper lanes hand their values
// to the lower ones through shared memory (xch, 64 rows of BN + 1 floats at the
// start of the ring, which nothing reads any more).  All eight epilogue warps meet at the
// barrier, whether their wait for the accumulator ran out or not.
template <int BN>
__device__ __forceinline__ void store_swiglu_half(uint32_t taddr, int q, int lane, int hgrp,
                                                  bool ok, float *xch,
                                                  bf16 *__restrict__ out_act, int m0, int ff,
                                                  int n0, int n)
{
    constexpr int LD = BN + 1;
    float v[16];
    if (ok && q >= 2) {
        float *row = xch + ((q - 2) * 32 + lane) * LD;
        for (int c = 16 * hgrp; c < BN; c += 32) {
            tc_ld16(taddr + c, v);
#pragma unroll
            for (int j = 0; j < 16; j++)
                row[c + j] = v[j];
        }
    }
    named_barrier(1, GEMM_THREADS - 64);
    if (ok && q < 2) {
        int j0 = q * 32 + lane, f = m0 + j0;
        const float *row = xch + j0 * LD;
        for (int c = 16 * hgrp; c < BN; c += 32) {
            tc_ld16(taddr + c, v);
            if (f < ff) {
                bf16 *p = out_act + (size_t)(n0 + c) * ff + f;
#pragma unroll
                for (int j = 0; j < 16; j++, p += ff)
                    if (n0 + c + j < n) {
                        float gv = v[j], uv = row[c + j];
                        float e = fast_exp2(gv * -1.4426950408889634f);
                        *p = __float2bfloat16_rn(__fdividef(gv * uv, 1.0f + e));
                    }
            }
        }
    }
}

template <int BN, int MT, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
               float *__restrict__ out, bf16 *__restrict__ out_act, int n, int m, int k,
               int second_off, int kb_per_split)
{
    using Cfg = TileCfg<BN, MT, EPI == EPI_SWIGLU_HALF>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = (uint64_t *)(smem + STAGES * Cfg::STAGE_BYTES);
    // bars[0..STAGES): full; [STAGES..2 STAGES): empty; [2 STAGES]: accumulator ready
    uint32_t *tmem_slot = (uint32_t *)(bars + 2 * STAGES + 1);
    volatile int *abort = (volatile int *)(tmem_slot + 1);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_w);
        prefetch_tensor_map(&map_a);
    }
    // token tiles vary fastest: the CTAs that run at the same time share weight
    // tiles, which then come from memory once, and the (small) activations come
    // from the L2
    int m0 = blockIdx.y * (EPI == EPI_SWIGLU ? TILE_M : EPI == EPI_SWIGLU_HALF ? HALF_M
                                                                                : TILE_M * MT);
    int n0 = blockIdx.x * BN;
    int total_kb = (k + BK - 1) / BK;
    int kb0 = blockIdx.z * kb_per_split;
    int nkb = min(kb_per_split, total_kb - kb0);

    uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES),
             accum = smem_u32(bars + 2 * STAGES);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum, 1);
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem = *tmem_slot;

    pdl_trigger();
    if (warp == 0 && lane == 0 && nkb > 0) {
        // ---------------------------------------------------------- TMA loads
        // The weights do not depend on the kernel before this one: their first
        // stages are on their way before that kernel has finished.  The
        // activations do: they are loaded after the dependency wait.
        uint32_t armed = 0, last_parity = 0;
        // a stage's weight tiles: MT boxes of 128 rows, or (EPI_SWIGLU_HALF) two boxes
        // of 64 rows, the gate's and the up projection's, that make one tile
        auto load_w = [&](uint32_t dst, uint32_t bar, int kx) {
            if (EPI == EPI_SWIGLU_HALF) {
                tma_load_2d(dst, &map_w, bar, kx, m0);
                tma_load_2d(dst + W_TILE_BYTES / 2, &map_w, bar, kx, m0 + second_off);
            } else {
#pragma unroll
                for (int t = 0; t < MT; t++)
                    tma_load_2d(dst + t * W_TILE_BYTES, &map_w, bar, kx, m0 + t * second_off);
            }
        };
        int pre = min(nkb, STAGES);
        for (int i = 0; i < pre; i++) {
            uint32_t dst = smem_u32(smem + i * Cfg::STAGE_BYTES);
            uint32_t bar = full0 + 8 * i;
            mbar_expect_tx(bar, Cfg::STAGE_BYTES);
            load_w(dst, bar, (kb0 + i) * BK);
            armed |= 1u << i;
        }
        pdl_wait();
        for (int i = 0; i < pre; i++)
            tma_load_2d(smem_u32(smem + i * Cfg::STAGE_BYTES) + MT * W_TILE_BYTES, &map_a,
                        full0 + 8 * i, (kb0 + i) * BK, n0);
        for (int i = pre; i < nkb; i++) {
            int s = i % STAGES;
            uint32_t ph = (i / STAGES) & 1;
            if (!mbar_wait(empty0 + 8 * s, ph ^ 1, abort, &g_gemm_tc_error, 1))
                break;
            uint32_t dst = smem_u32(smem + s * Cfg::STAGE_BYTES);
            uint32_t bar = full0 + 8 * s;
            mbar_expect_tx(bar, Cfg::STAGE_BYTES);
            int kx = (kb0 + i) * BK;
            load_w(dst, bar, kx);
            tma_load_2d(dst + MT * W_TILE_BYTES, &map_a, bar, kx, n0);
            armed |= 1u << s;
            last_parity = (last_parity & ~(1u << s)) | (ph << s);
        }
        if (*abort) {
            // the loads in flight: wait for each stage armed last, once, with the limit
            volatile int never = 0;
            for (int s = 0; s < STAGES; s++)
                if (armed & (1u << s))
                    mbar_wait(full0 + 8 * s, (last_parity >> s) & 1, &never, &g_gemm_tc_error, 4);
        }
    } else if (warp == 1 && lane == 0 && nkb > 0) {
        // --------------------------------------------------------------- MMAs
        constexpr uint32_t idesc = instr_desc(BN);
        bool ok = true;
        for (int i = 0; i < nkb && ok; i++) {
            int s = i % STAGES;
            uint32_t ph = (i / STAGES) & 1;
            ok = mbar_wait(full0 + 8 * s, ph, abort, &g_gemm_tc_error, 2);
            if (!ok)
                break;
            tc_fence_after();
            uint32_t base = smem_u32(smem + s * Cfg::STAGE_BYTES);
            uint64_t da = smem_desc(base + MT * W_TILE_BYTES);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                uint64_t dw = smem_desc(base + t * W_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++)
                    tc_mma(tmem + t * BN, dw + 2 * kk, da + 2 * kk, idesc, (i | kk) != 0);
            }
            tc_commit(empty0 + 8 * s);
        }
        tc_commit(accum);
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue
        int q = warp & 3;                       // the TMEM lanes this warp may read
        int f = m0 + q * 32 + lane;             // this thread's feature (of tile 0)
        pdl_wait();                         // no store before the kernel before this one is done
        bool ok = nkb > 0 && mbar_wait(accum, 0, abort, &g_gemm_tc_error, 3);
        ok = __all_sync(0xffffffffu, ok);   // the TMEM loads below are warp-wide
        tc_fence_after();
        uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
        // The accumulator is read 32 columns (tokens) at a time; the read of the
        // next 32 is in flight while the last 32 are stored.
        int hgrp = (warp - 2) >> 2;             // which of the two warps of this quarter
        if (EPI == EPI_SWIGLU_HALF) {
            if constexpr (MT == 1 && BN <= 128)
                store_swiglu_half<BN>(taddr, q, lane, hgrp, ok, (float *)smem, out_act, m0,
                                      second_off, n0, n);
        } else if (ok) {
            if (EPI == EPI_PARTIAL)
                store_partial<BN, MT>(taddr, hgrp, out + (size_t)blockIdx.z * n * m, f, n0, n, m,
                                      second_off);
            else
                store_swiglu<BN>(taddr, hgrp, out_act, f, second_off, n0, n);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
EncodeTiled tensor_map_encoder()
{
    static EncodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    });
    return fn;
}

// A [rows, k] bfloat16 row-major matrix, read in boxes of box_rows x 64 with the
// 128-byte swizzle; what lies outside the matrix reads as zero.
static bool tensor_map(const void *ptr, int rows, int k, int box_rows, CUtensorMap *out)
{
    typedef std::tuple<const void *, int, int, int> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    Key key(ptr, rows, k, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiled enc = tensor_map_encoder();
    if (!enc)
        return false;
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap map;
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(ptr), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 8192)
        cache.clear();
    cache[key] = map;
    *out = map;
    return true;
}

template <int BN, int MT, int EPI>
static int launch_tc(const void *A, const void *W, float *out, bf16 *out_act, int n, int m, int k,
                     int w_rows, int second_off, int splits, cudaStream_t st)
{
    using Cfg = TileCfg<BN, MT, EPI == EPI_SWIGLU_HALF>;
    CUtensorMap map_w, map_a;
    if (!tensor_map(W, w_rows, k, EPI == EPI_SWIGLU_HALF ? HALF_M : TILE_M, &map_w) ||
        !tensor_map(A, n, k, BN, &map_a))
        return JB_EINVAL;
    auto kern = gemm_tc_kernel<BN, MT, EPI>;
    static unsigned long long smem_allowed = 0;
    if (!allow_dynamic_smem(kern, Cfg::SMEM_BYTES, smem_allowed))
        return JB_ELAUNCH;
    int total_kb = (k + BK - 1) / BK;
    int kbps = (total_kb + splits - 1) / splits;
    if ((splits - 1) * kbps >= total_kb)
        return JB_EINVAL;   // a part without work
    int feats = EPI == EPI_PARTIAL ? m : second_off;
    int tile_feats = EPI == EPI_SWIGLU ? TILE_M : EPI == EPI_SWIGLU_HALF ? HALF_M : TILE_M * MT;
    dim3 grid((n + BN - 1) / BN, (feats + tile_feats - 1) / tile_feats, splits);
    if (grid.y > 65535 || grid.z > 65535)
        return JB_EINVAL;
    launch(kern, grid, GEMM_THREADS, Cfg::SMEM_BYTES, st, map_w, map_a, out, out_act, n, m, k, second_off,
           kbps);
    return launch_status();
}

}  // namespace jb

using namespace jb;

// Whether the tensor-core product takes this shape: bfloat16 rows whose length
// is a multiple of 8 (TMA wants 16-byte strides), 16-byte aligned bases.
extern "C" int jb_gemm_tc_ok(const void *A, const void *W, int n, int m, int k)
{
    return n > 0 && m > 0 && k >= 8 && k % 8 == 0 && (uintptr_t)A % 16 == 0 &&
           (uintptr_t)W % 16 == 0;
}

// Parts of k that a product of this shape is best cut into (>= 1).  With few
// tokens the product is a stream of weights, and what one CTA pulls is limited
// by the loads it can keep in flight: measured on B200, the products of a
// decode step run fastest when their CTAs (feature tiles x parts of k) just
// fill the SMs' places for this kernel (two a SM) at once, as long as a part
// keeps at least four 64-wide blocks of k.  More CTAs than places come in waves
// whose last one straggles, so a product with more tiles than that is not cut.
static int many_tokens_splits(int n, int m, int k);

extern "C" int jb_gemm_tc_splits(int n, int m, int k)
{
    if (n > 128)
        return many_tokens_splits(n, m, k);
    const int PLACES = 2 * sm_count();
    int bn = n <= 16 ? 16 : n <= 32 ? 32 : n <= 64 ? 64 : 128;
    long tiles = (long)((m + TILE_M - 1) / TILE_M) * ((n + bn - 1) / bn);
    int total_kb = (k + BK - 1) / BK;
    int best = 1;
    for (int s = 2; s <= 16 && tiles * s <= PLACES; s++) {
        int kbps = (total_kb + s - 1) / s;
        if (kbps < 4)
            break;
        if ((s - 1) * kbps >= total_kb)
            continue;                              // a part without work
        best = s;
    }
    return best;
}

// Tokens per tile (256 features x this many tokens) for a product over many
// tokens whose k is cut into `splits` parts, and the estimate of its time in
// microseconds.  One CTA fits an SM, so tiles run in rounds of as many as there
// are SMs; a narrower tile can turn a mostly empty last round into none.  A
// tile's time is a fixed part plus, per 64-wide block of k, the larger of its MMA
// time and the time to bring its operands in (measured: about 116 GB/s per SM),
// which is why narrower tiles are not proportionally faster.  Every part beyond
// the first also costs the writing and the reading back of a float partial sum.
static int many_tokens_tile_choice(int n, int m, int k, int splits, double *time_us);
static int g_forced_tile = 0;   // tokens per tile that the next products must take; 0: the choice below
static int g_last_tile = 0;     // what the last product over many tokens took

static int many_tokens_tile(int n, int m, int k, int splits, double *time_us = nullptr)
{
    if (g_forced_tile && !time_us)
        return g_last_tile = g_forced_tile;
    int best = many_tokens_tile_choice(n, m, k, splits, time_us);
    if (!time_us)
        g_last_tile = best;
    return best;
}

// For tests: makes every product over more than 128 tokens take tiles of this many
// tokens (128, 160, 192, 224 or 256; 0: the library's own choice again), and says
// which width the last such product took.  Every width computes the same sums; the
// choice is one of speed.
extern "C" int jb_gemm_tc_force_tile(int tokens)
{
    if (tokens != 0 && tokens != 128 && tokens != 160 && tokens != 192 && tokens != 224 && tokens != 256)
        return JB_EINVAL;
    g_forced_tile = tokens;
    return JB_OK;
}
extern "C" int jb_gemm_tc_last_tile(void) { return g_last_tile; }

static int many_tokens_tile_choice(int n, int m, int k, int splits, double *time_us)
{
    int sms = sm_count();
    const int choices[5] = {256, 224, 192, 160, 128};
    int kb = (k + BK - 1) / BK;
    int kbps = (kb + splits - 1) / splits;
    long m_tiles = (m + 2 * TILE_M - 1) / (2 * TILE_M);
    int best = 256;
    double best_t = 1e30;
    for (int c = 0; c < 5; c++) {
        int bn = choices[c];
        long tiles = m_tiles * ((n + bn - 1) / bn) * splits;
        long rounds = (tiles + sms - 1) / sms;
        double mma = 0.55 * bn / 256.0, load = (32768.0 + bn * 128.0) / 116000.0;
        // tiles above 192 tokens have room for three stages only, two of them in
        // flight: measured, a block of k then takes a fifth longer than its bytes do
        if (bn > 192)
            load *= 1.2;
        double t = rounds * (8.0 + kbps * (mma > load ? mma : load)) +
                   (splits - 1) * (double)n * m * 8.0 / 5e6;
        if (t < best_t * 0.98) {
            best_t = t;
            best = bn;
        }
    }
    if (time_us)
        *time_us = best_t;
    return best;
}

// Parts of k for a product over many tokens: more than one only where the tiles
// alone leave most SMs idle (a few hundred tokens times a narrow weight matrix).
static int many_tokens_splits(int n, int m, int k)
{
    int kb = (k + BK - 1) / BK;
    int best = 1;
    double best_t = 1e30;
    for (int s = 1; s <= 8; s++) {
        int kbps = (kb + s - 1) / s;
        if (s > 1 && (kbps < 8 || (s - 1) * kbps >= kb))
            continue;
        double t;
        many_tokens_tile(n, m, k, s, &t);
        if (t < best_t * 0.95) {
            best_t = t;
            best = s;
        }
    }
    return best;
}

// out: [splits, n, m] float partial sums of A[n, k] . W[m, k]^T.
extern "C" int jb_gemm_tc(const void *A, const void *W, float *out, int n, int m, int k, int splits,
                          cudaStream_t st)
{
    if (!jb_gemm_tc_ok(A, W, n, m, k) || splits < 1)
        return JB_EINVAL;
    if (n > 128) {
#define JB_MANY(B) launch_tc<B, 2, EPI_PARTIAL>(A, W, out, nullptr, n, m, k, m, TILE_M, splits, st)
        switch (many_tokens_tile(n, m, k, splits)) {
        case 128: return JB_MANY(128);
        case 160: return JB_MANY(160);
        case 192: return JB_MANY(192);
        case 224: return JB_MANY(224);
        default: return JB_MANY(256);
        }
#undef JB_MANY
    }
    if (n <= 16)
        return launch_tc<16, 1, EPI_PARTIAL>(A, W, out, nullptr, n, m, k, m, TILE_M, splits, st);
    if (n <= 32)
        return launch_tc<32, 1, EPI_PARTIAL>(A, W, out, nullptr, n, m, k, m, TILE_M, splits, st);
    if (n <= 64)
        return launch_tc<64, 1, EPI_PARTIAL>(A, W, out, nullptr, n, m, k, m, TILE_M, splits, st);
    return launch_tc<128, 1, EPI_PARTIAL>(A, W, out, nullptr, n, m, k, m, TILE_M, splits, st);
}

// W: [2 ff, k], rows [0, ff) the gate and [ff, 2 ff) the up projection.
// out_act[n, ff] = SiLU(A . gate^T) * (A . up^T) in bfloat16.
extern "C" int jb_gemm_tc_swiglu(const void *A, const void *W, void *out_act, int n, int ff, int k,
                                 cudaStream_t st)
{
    if (!jb_gemm_tc_ok(A, W, n, 2 * ff, k))
        return JB_EINVAL;
    if (n > 128) {
#define JB_SWIGLU(B)                                                                           \
    launch_tc<B, 2, EPI_SWIGLU>(A, W, nullptr, (bf16 *)out_act, n, 2 * ff, k, 2 * ff, ff, 1, st)
        switch (many_tokens_tile(n, 2 * ff, k, 1)) {
        case 128: return JB_SWIGLU(128);
        case 160: return JB_SWIGLU(160);
        case 192: return JB_SWIGLU(192);
        case 224: return JB_SWIGLU(224);
        default: return JB_SWIGLU(256);
        }
#undef JB_SWIGLU
    }
    // few tokens: as many CTAs as the plain product has (64 gate and 64 up features each)
#define JB_SWIGLU_HALF(B)                                                                      \
    launch_tc<B, 1, EPI_SWIGLU_HALF>(A, W, nullptr, (bf16 *)out_act, n, 2 * ff, k, 2 * ff, ff, 1, st)
    if (n <= 16)
        return JB_SWIGLU_HALF(16);
    if (n <= 32)
        return JB_SWIGLU_HALF(32);
    if (n <= 64)
        return JB_SWIGLU_HALF(64);
    return JB_SWIGLU_HALF(128);
#undef JB_SWIGLU_HALF
}

// Reads and clears the error word: 0, or which wait ran out first (1: a free
// stage, 2: a loaded stage, 3: the accumulator, 4: a load in flight).
// Synchronizes the device.
// A wait that nothing ends, to show that a bounded wait runs out as it should: one
// warp, one mbarrier that no thread and no copy ever arrives at, the products' own
// wait with a limit of limit_cycles.  The kernel returns when the limit has passed
// and leaves code 9 in the products' error word (jb_gemm_tc_error reads and clears
// it).  Nothing faults and nothing is left waiting.
__global__ void wait_selftest_kernel(long long limit_cycles)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0)
        mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, &g_gemm_tc_error, 9, limit_cycles);
}

// Runs the kernel above and waits for it; limit_cycles is cut to 20 million (about
// ten milliseconds).  Returns 0, or JB_ELAUNCH.
extern "C" int jb_wait_selftest(long long limit_cycles)
{
    if (limit_cycles < 1000)
        limit_cycles = 1000;
    if (limit_cycles > 20000000ll)
        limit_cycles = 20000000ll;
    wait_selftest_kernel<<<1, 32>>>(limit_cycles);
    if (cudaGetLastError() != cudaSuccess)
        return JB_ELAUNCH;
    return cudaDeviceSynchronize() == cudaSuccess ? JB_OK : JB_ELAUNCH;
}

extern "C" int jb_gemm_tc_error(void)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_tc_error, sizeof v) != cudaSuccess)
        return JB_ELAUNCH;
    if (v != 0)
        cudaMemcpyToSymbol(g_gemm_tc_error, &zero, sizeof zero);
    return v;
}
