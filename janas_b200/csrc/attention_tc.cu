// Causal grouped-query attention over the paged cache on the tensor cores
// (tcgen05), for bfloat16 heads of 64 or 128 values.  Keys and values come in
// chunks of 128 positions, two cache pages, straight from the pages into shared
// memory by TMA; V is read as an MN-major operand as it lies in the page
// ([position][value]).  Three kernels:
//
// attn_tc_prefill_kernel   A CTA works for one KV head on two blocks of 128 rows:
//     the G query heads of the group for 2 R consecutive positions of one
//     sequence (R = 128 / G a block).  Per chunk and block S = Q K^T, softmax by
//     one thread per row (scale, causal and window mask, exp, sum; P to shared
//     memory in bfloat16), O += P V with O in tensor memory; the blocks take
//     turns on the tensor core and share the chunk's keys and values.
//
// attn_tc_decode_kernel    One decoded token, heads of 128 values, up to 16
//     heads per KV head: the keys are the M operand (S^T = K Q^T, O^T = V^T P),
//     one thread per key; a CTA runs over its chunks and leaves one partial
//     (m, l, O) per head, which attention.cu's merge kernel joins.  That spreads
//     one token's long context over many SMs.
//
// attn_tc_rows_kernel      One decoded token for the sizes the kernel above does
//     not take (heads of 64 values, more than 16 heads per KV head): the block
//     of 128 rows holds the group's heads, one chunk per CTA, one partial per
//     chunk.
//
// Warp 0 issues the TMA loads, warp 1 owns the tensor memory and issues the
// MMAs, the other warps are the row (or key) threads.  Every mbarrier wait has a
// time limit (see tc_common.cuh); a wait that runs out is recorded in an error
// word (jb_attn_tc_error) and the CTA winds down.  No load uses cluster
// multicast.
//
// Formulas as in attention.cu (reference: src/llm/attention.c:107-118,574-588,
// 734-739,870-910).
#include <map>
#include <mutex>
#include <tuple>

#include "kernels.h"
#include "tc_common.cuh"

namespace jb {

constexpr int AT_ROWS = 128;        // rows of a block (TMEM lanes)
constexpr int AT_KEYS = 128;        // keys per chunk (= ATT_CHUNK of attention.cu)
constexpr int AT_STAGES = 2;        // K/V chunks in flight
constexpr int BLK_BYTES = 128 * 128;  // a 128-row block of 64 bfloat16 columns

__device__ int g_attn_tc_error;

template <int HD> struct AttnCfg {
    static constexpr int NB = HD / 64;                 // 64-column blocks per head
    static constexpr int Q_BYTES = NB * BLK_BYTES;
    static constexpr int P_BYTES = 2 * BLK_BYTES;      // 128 rows x 128 keys
    static constexpr int KV_STAGE = 2 * NB * BLK_BYTES;  // K and V of one chunk
    static constexpr int SMEM_BYTES = Q_BYTES + P_BYTES + AT_STAGES * KV_STAGE + 1024 + 2048;
    static constexpr int TMEM_COLS = 256;              // S: 128 columns, PV: HD <= 128
};

// Byte offset of (row, 16-byte chunk j of the row's 128 bytes) inside a block of
// 128-byte rows in the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int row, int j)
{
    return (uint32_t)(row * 128 + ((j ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(192)
attn_tc_rows_kernel(const __grid_constant__ CUtensorMap map_q,
                    const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v,
                    const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                    const int32_t *__restrict__ block_table, int bt_stride,
                    float *__restrict__ part, int nh, int nkv, int G, int window, float scale,
                    int max_chunks, int chunks_per_cta, int row0)
{
    using Cfg = AttnCfg<HD>;
    constexpr int NB = Cfg::NB;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem;
    uint8_t *p_s = q_s + Cfg::Q_BYTES;
    uint8_t *kv_s = p_s + Cfg::P_BYTES;
    uint64_t *bars = (uint64_t *)(kv_s + AT_STAGES * Cfg::KV_STAGE);
    // bars: 0 q_full | 1,2 kv_full | 3,4 kv_empty | 5 s_full | 6 p_full | 7 o_full | 8 pv_free
    uint32_t *tmem_slot = (uint32_t *)(bars + 9);
    volatile int *abort = (volatile int *)(tmem_slot + 1);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int kvh = blockIdx.y;

    // ---- what this CTA works on: a run of chunks of one decoded token
    int parts = (max_chunks + chunks_per_cta - 1) / chunks_per_cta;
    int lrow = blockIdx.x / parts, part_i = blockIdx.x % parts;
    int q_row = row0 + lrow;
    int q_pos = row_pos[q_row];
    int seq = row_seq[q_row];
    int lo = window > 0 && q_pos + 1 > window ? q_pos + 1 - window : 0;
    int c_base = lo / AT_KEYS;         // the row's first chunk (index 0 of its partials)
    int c_first = c_base + part_i * chunks_per_cta;
    int c_last = min(q_pos / AT_KEYS, c_first + chunks_per_cta - 1);
    int n_chunks = c_last - c_first + 1;
    if (n_chunks <= 0)
        return;                        // nothing to do: before any barrier or tensor memory

    uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8 * i; };
    if (threadIdx.x == 0) {
        mbar_init(bar(0), 1);
        for (int s = 0; s < AT_STAGES; s++) {
            mbar_init(bar(1 + s), 1);
            mbar_init(bar(3 + s), 1);
        }
        mbar_init(bar(5), 1);
        mbar_init(bar(6), AT_ROWS);
        mbar_init(bar(7), 1);
        mbar_init(bar(8), AT_ROWS);
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
    uint32_t tmem_s = tmem, tmem_pv = tmem + AT_KEYS;
    int *err = &g_attn_tc_error;
    // q, the keys and the values were written by the kernel before this one
    pdl_trigger();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- TMA loads
        mbar_expect_tx(bar(0), (uint32_t)(G * HD * 2));
#pragma unroll
        for (int b = 0; b < NB; b++)
            tma_load_3d(smem_u32(q_s + b * BLK_BYTES), &map_q, bar(0), b * 64, kvh * G, q_row);
        const int32_t *bt = block_table + (size_t)seq * bt_stride;
        uint32_t armed = 0, last_parity = 0;
        for (int it = 0; it < n_chunks; it++) {
            int s = it % AT_STAGES;
            uint32_t ph = (it / AT_STAGES) & 1;
            if (!mbar_wait(bar(3 + s), ph ^ 1, abort, err, 1))
                break;
            mbar_expect_tx(bar(1 + s), Cfg::KV_STAGE);
            uint32_t k_dst = smem_u32(kv_s + s * Cfg::KV_STAGE);
            uint32_t v_dst = k_dst + NB * BLK_BYTES;
            int c = c_first + it;
#pragma unroll
            for (int pg = 0; pg < 2; pg++) {
                int idx = 2 * c + pg;
                int page = idx < bt_stride ? bt[idx] : -1;
                if (page < 0)
                    page = 0;          // not there: every position of it is masked
                int y = (page * nkv + kvh) * PAGE;
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    tma_load_2d(k_dst + b * BLK_BYTES + pg * (PAGE * 128), &map_k, bar(1 + s),
                                b * 64, y);
                    tma_load_2d(v_dst + b * BLK_BYTES + pg * (PAGE * 128), &map_v, bar(1 + s),
                                b * 64, y);
                }
            }
            armed |= 1u << s;
            last_parity = (last_parity & ~(1u << s)) | (ph << s);
        }
        if (*abort) {
            volatile int never = 0;
            for (int s = 0; s < AT_STAGES; s++)
                if (armed & (1u << s))
                    mbar_wait(bar(1 + s), (last_parity >> s) & 1, &never, err, 4);
        }
    } else if (warp == 1 && lane == 0) {
        // --------------------------------------------------------------- MMAs
        constexpr uint32_t idesc_s = instr_desc_bf16(AT_ROWS, AT_KEYS, false);
        constexpr uint32_t idesc_pv = instr_desc_bf16(AT_ROWS, HD, true);
        bool ok = mbar_wait(bar(0), 0, abort, err, 2);
        uint32_t q_a = smem_u32(q_s), p_a = smem_u32(p_s);
        for (int it = 0; it < n_chunks && ok; it++) {
            int s = it % AT_STAGES;
            uint32_t ph = (it / AT_STAGES) & 1;
            ok = mbar_wait(bar(1 + s), ph, abort, err, 3);
            if (!ok)
                break;
            tc_fence_after();
            uint32_t k_a = smem_u32(kv_s + s * Cfg::KV_STAGE);
            uint32_t v_a = k_a + NB * BLK_BYTES;
            // S = Q K^T over the head's values, 16 at a time
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
                uint32_t off = (kk / 4) * BLK_BYTES + (kk % 4) * 32;
                tc_mma(tmem_s, smem_desc_sw128(q_a + off, 16, 1024),
                       smem_desc_sw128(k_a + off, 16, 1024), idesc_s, kk != 0);
            }
            tc_commit(bar(5));
            ok = mbar_wait(bar(6), it & 1, abort, err, 5);       // P is in shared memory
            if (ok && it > 0)
                ok = mbar_wait(bar(8), (it - 1) & 1, abort, err, 6);   // the last PV was read
            if (!ok)
                break;
            tc_fence_after();
            // PV = P V over the chunk's keys, 16 at a time; V is MN-major: blocks of 64
            // values BLK_BYTES apart, groups of eight keys 1024 bytes apart
#pragma unroll
            for (int kk = 0; kk < AT_KEYS / 16; kk++) {
                uint32_t p_off = (kk / 4) * BLK_BYTES + (kk % 4) * 32;
                tc_mma(tmem_pv, smem_desc_sw128(p_a + p_off, 16, 1024),
                       smem_desc_sw128(v_a + kk * 16 * 128, BLK_BYTES, 1024), idesc_pv, kk != 0);
            }
            tc_commit(bar(7));
            tc_commit(bar(3 + s));
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ row threads
        int qw = warp & 3;                      // the TMEM lanes this warp may read
        int r = qw * 32 + lane;                 // this thread's row of the block
        int g = r;                              // the head of the group
        bool live = r < G;
        bool warp_live = __any_sync(0xffffffffu, live);
        int pos = q_pos;
        uint32_t lane_addr = (uint32_t)(qw * 32) << 16;
        const float c2 = scale * 1.4426950408889634f;      // scores in units of log2(e)
        bool ok = true;
        for (int it = 0; it < n_chunks; it++) {
            int c = c_first + it;
            int t0 = c * AT_KEYS;
            ok = ok && mbar_wait(bar(5), it & 1, abort, err, 7);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            float m_new = -INFINITY, l_chunk = 0.0f;   // every chunk is a partial of its own
            if (ok && warp_live) {
                // first pass: the largest visible score of the chunk
                float mx = -INFINITY;
#pragma unroll 1
                for (int cb = 0; cb < AT_KEYS / 32; cb++) {
                    float sc[32];
                    tc_ld32(tmem_s + lane_addr + cb * 32, sc);
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        int t = t0 + cb * 32 + i;
                        if (live && t <= pos && t >= lo)
                            mx = fmaxf(mx, sc[i] * c2);
                    }
                }
                m_new = mx;
                // second pass: the weights, their sum, and P in bfloat16
#pragma unroll 1
                for (int cb = 0; cb < AT_KEYS / 32; cb++) {
                    float sc[32];
                    tc_ld32(tmem_s + lane_addr + cb * 32, sc);
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        int t = t0 + cb * 32 + i;
                        float p0 = (live && t <= pos && t >= lo) ? exp2f(sc[i] * c2 - m_new) : 0.0f;
                        float p1 = (live && t + 1 <= pos && t + 1 >= lo)
                                       ? exp2f(sc[i + 1] * c2 - m_new) : 0.0f;
                        l_chunk += p0 + p1;
                        __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                        packed[i / 2] = *reinterpret_cast<uint32_t *>(&pk);
                    }
                    // 32 keys = 64 bytes = four 16-byte chunks of this row
                    uint8_t *blk = p_s + (cb / 2) * BLK_BYTES;
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        uint4 v = make_uint4(packed[4 * q4], packed[4 * q4 + 1],
                                             packed[4 * q4 + 2], packed[4 * q4 + 3]);
                        *reinterpret_cast<uint4 *>(blk + swz(r, (cb % 2) * 4 + q4)) = v;
                    }
                }
            } else if (ok) {
                // an idle warp's rows of P must still be finite: zero them once
                if (it == 0) {
#pragma unroll 1
                    for (int b = 0; b < 2; b++)
#pragma unroll
                        for (int q8 = 0; q8 < 8; q8++)
                            *reinterpret_cast<uint4 *>(p_s + b * BLK_BYTES + swz(r, q8)) =
                                make_uint4(0, 0, 0, 0);
                }
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(bar(6));
            ok = ok && mbar_wait(bar(7), it & 1, abort, err, 8);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            if (ok && warp_live) {
                float *dst = nullptr;
                if (live) {
                    size_t at = (((size_t)lrow * nh + kvh * G + g) * max_chunks + (c - c_base)) *
                                (size_t)(HD + 2);
                    dst = part + at;
                    // the merge works with exp(): natural-log units
                    dst[0] = m_new * 0.6931471805599453f;
                    dst[1] = l_chunk;
                }
#pragma unroll 1
                for (int db = 0; db < HD / 32; db++) {
                    float pv[32];
                    tc_ld32(tmem_pv + lane_addr + db * 32, pv);
                    if (live) {
#pragma unroll
                        // a partial is hd + 2 floats long: 8-byte aligned, not 16
                        for (int i = 0; i < 32; i += 2)
                            *reinterpret_cast<float2 *>(dst + 2 + db * 32 + i) =
                                make_float2(pv[i], pv[i + 1]);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar(8));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// --------------------------------------------------------------- prefill rows
// A CTA works for one KV head on two blocks of 128 rows, A and B: the G query
// heads of the group for 2 R consecutive positions of one sequence (R = 128 / G
// each).  Both blocks use the same keys and values, so a chunk is loaded once for
// 256 rows, and they take turns: while one block's row threads turn scores into
// weights, the tensor core works on the other block.  One thread per row: no
// exchange between threads.
//
//   per chunk and block:  S = Q K^T  ->  row thread: S from tensor memory, mask,
//   maximum, p = 2^(s - m), sum, P to shared memory in bfloat16  ->  O += P V
//
// O stays in tensor memory and P V accumulates onto it.  A row's exponent
// reference m is therefore not moved with every chunk but only when the chunk's
// maximum exceeds it by more than 8 (weights up to 2^8, far inside bfloat16 and
// float range); then the row thread scales its row of O and its sum by
// 2^(m_old - m_new) before it hands P over.  After the first chunks that is rare.
//
// Tensor memory: S_A [0, 128), S_B [128, 256), O_A [256, 256 + HD), O_B after it.
// Shared memory: Q_A, Q_B, P_A, P_B, and a ring of three units that hold keys and
// values in the order of their use: K0 K1 V0 K2 V1 K3 ...
constexpr int PF_THREADS = 320;     // warp 0 loads, warp 1 issues MMAs, 2..5 rows of A, 6..9 of B
constexpr int PF_UNITS = 3;
constexpr float PF_LAZY = 8.0f;     // how far (in powers of two) a maximum may run ahead of m

template <int HD> struct PrefillCfg {
    static constexpr int NB = HD / 64;
    static constexpr int Q_TILE = NB * BLK_BYTES;          // 128 rows x HD
    static constexpr int P_TILE = 2 * BLK_BYTES;           // 128 rows x 128 keys
    static constexpr int UNIT = NB * BLK_BYTES;            // 128 positions x HD
    static constexpr int TAIL = 3072;                      // barriers and the like
    static constexpr int SMEM_BYTES = 2 * Q_TILE + 2 * P_TILE + PF_UNITS * UNIT + TAIL;
    static constexpr int TMEM_COLS = 512;
};

template <int HD>
__global__ void __launch_bounds__(PF_THREADS, 1)
attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int32_t *__restrict__ qblk,
                       const int32_t *__restrict__ block_table, int bt_stride,
                       bf16 *__restrict__ out, int nh, int nkv, int G, int R, int window,
                       float scale)
{
    using Cfg = PrefillCfg<HD>;
    constexpr int NB = Cfg::NB;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *q_s = smem;                           // two tiles
    uint8_t *p_s = q_s + 2 * Cfg::Q_TILE;          // two tiles
    uint8_t *kv_s = p_s + 2 * Cfg::P_TILE;
    uint64_t *bars = (uint64_t *)(kv_s + PF_UNITS * Cfg::UNIT);
    // bars: 0 q_full | 1..3 unit full | 4..6 unit free | 7,8 s_full A,B | 9,10 p_full A,B |
    //       11,12 pv_done A,B | 13,14 s_free A,B
    uint32_t *tmem_slot = (uint32_t *)(bars + 15);
    volatile int *abort = (volatile int *)(tmem_slot + 1);

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_q);
        prefetch_tensor_map(&map_k);
        prefetch_tensor_map(&map_v);
    }
    // qblk lists the longest runs first; all KV heads of a run are neighbours in the
    // grid, so that CTAs start in the order of their length
    int kvh = blockIdx.x % nkv;
    const int32_t *b = qblk + 4 * (blockIdx.x / nkv);
    int q_row = b[0], q_count = b[1], q_pos = b[2], seq = b[3];
    bool has_b = q_count > R;                                    // the second block has rows
    int lo0 = window > 0 && q_pos + 1 > window ? q_pos + 1 - window : 0;
    int c_first = lo0 / AT_KEYS;
    int c_last = (q_pos + q_count - 1) / AT_KEYS;
    int n_chunks = c_last - c_first + 1;
    if (n_chunks <= 0)
        return;

    uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8 * i; };
    if (threadIdx.x == 0) {
        mbar_init(bar(0), 1);
        for (int s = 0; s < PF_UNITS; s++) {
            mbar_init(bar(1 + s), 1);
            mbar_init(bar(4 + s), 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(bar(7 + t), 1);
            mbar_init(bar(9 + t), AT_ROWS);
            mbar_init(bar(11 + t), 1);
            mbar_init(bar(13 + t), AT_ROWS);
        }
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
    int *err = &g_attn_tc_error;
    // q, the keys and the values were written by the kernel before this one
    pdl_trigger();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- TMA loads
        mbar_expect_tx(bar(0), (uint32_t)((has_b ? 2 : 1) * R * G * HD * 2));
        for (int t = 0; t < (has_b ? 2 : 1); t++)
#pragma unroll
            for (int bb = 0; bb < NB; bb++)
                tma_load_3d(smem_u32(q_s + t * Cfg::Q_TILE + bb * BLK_BYTES), &map_q, bar(0),
                            bb * 64, kvh * G, q_row + t * R);
        const int32_t *bt = block_table + (size_t)seq * bt_stride;
        uint32_t armed = 0, last_parity = 0;
        for (int u = 0; u < 2 * n_chunks; u++) {       // units in the order they are used
            int s = u % PF_UNITS;
            uint32_t ph = (u / PF_UNITS) & 1;
            if (!mbar_wait(bar(4 + s), ph ^ 1, abort, err, 21))
                break;
            mbar_expect_tx(bar(1 + s), Cfg::UNIT);
            uint32_t dst = smem_u32(kv_s + s * Cfg::UNIT);
            bool is_v = u == 2 * n_chunks - 1 || (u > 0 && (u & 1) == 0);
            int chunk = u == 0 ? 0 : u == 2 * n_chunks - 1 ? n_chunks - 1 : is_v ? (u - 2) / 2
                                                                            : (u + 1) / 2;
            const CUtensorMap *map = is_v ? &map_v : &map_k;
            int c = c_first + chunk;
#pragma unroll
            for (int pg = 0; pg < 2; pg++) {
                int idx = 2 * c + pg;
                int page = idx < bt_stride ? bt[idx] : -1;
                if (page < 0)
                    page = 0;          // not there: every position of it is masked
                int y = (page * nkv + kvh) * PAGE;
#pragma unroll
                for (int bb = 0; bb < NB; bb++)
                    tma_load_2d(dst + bb * BLK_BYTES + pg * (PAGE * 128), map, bar(1 + s), bb * 64, y);
            }
            armed |= 1u << s;
            last_parity = (last_parity & ~(1u << s)) | (ph << s);
        }
        if (*abort) {
            volatile int never = 0;
            for (int s = 0; s < PF_UNITS; s++)
                if (armed & (1u << s))
                    mbar_wait(bar(1 + s), (last_parity >> s) & 1, &never, err, 24);
        }
    } else if (warp == 1 && lane == 0) {
        // --------------------------------------------------------------- MMAs
        constexpr uint32_t idesc_s = instr_desc_bf16(AT_ROWS, AT_KEYS, false);
        constexpr uint32_t idesc_pv = instr_desc_bf16(AT_ROWS, HD, true);
        int tiles = has_b ? 2 : 1;
        // The ring's units in the order of their use: K0, then for every chunk the next
        // chunk's keys before this chunk's values (K1 V0 K2 V1 ...), so that a unit is
        // asked for a whole chunk before it is needed.
        auto unit_k = [&](int j) { return j == 0 ? 0 : 2 * j - 1; };
        auto unit_v = [&](int j) { return j == n_chunks - 1 ? 2 * n_chunks - 1 : 2 * j + 2; };
        bool ok = mbar_wait(bar(0), 0, abort, err, 22);
        // the scores of chunk `it` of block t; the chunk's keys are in unit 2 it
        auto issue_s = [&](int it, int t) {
            // one descriptor per operand; the steps along k are added to its address
            // field (16-byte units), so that the one issuing thread has little to compute
            uint64_t dq = smem_desc_sw128(smem_u32(q_s + t * Cfg::Q_TILE), 16, 1024);
            uint64_t dk = smem_desc_sw128(
                smem_u32(kv_s + (unit_k(it) % PF_UNITS) * Cfg::UNIT), 16, 1024);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
                uint64_t off = (uint64_t)(((kk / 4) * BLK_BYTES + (kk % 4) * 32) >> 4);
                tc_mma(tmem + t * AT_KEYS, dq + off, dk + off, idesc_s, kk != 0);
            }
            tc_commit(bar(7 + t));
        };
        auto keys_there = [&](int it) {
            int u = unit_k(it);
            bool there = mbar_wait(bar(1 + u % PF_UNITS), (u / PF_UNITS) & 1, abort, err, 23);
            tc_fence_after();
            return there;
        };
        if (ok && (ok = keys_there(0))) {
            for (int t = 0; t < tiles; t++)
                issue_s(0, t);
            tc_commit(bar(4 + 0));                 // the keys' unit is free once these are done
        }
        for (int it = 0; it < n_chunks && ok; it++) {
            // the next chunk's scores as soon as the row threads hold this chunk's in
            // registers: they are there when the row threads come back for them
            if (it + 1 < n_chunks) {
                ok = keys_there(it + 1);
                for (int t = 0; t < tiles && ok; t++) {
                    ok = mbar_wait(bar(13 + t), it & 1, abort, err, 30);
                    if (!ok)
                        break;
                    tc_fence_after();
                    issue_s(it + 1, t);
                }
                if (!ok)
                    break;
                tc_commit(bar(4 + unit_k(it + 1) % PF_UNITS));
            }
            int uv = unit_v(it), sv = uv % PF_UNITS;
            for (int t = 0; t < tiles && ok; t++) {
                ok = mbar_wait(bar(9 + t), it & 1, abort, err, 25);               // P is there
                if (ok && t == 0)
                    ok = mbar_wait(bar(1 + sv), (uv / PF_UNITS) & 1, abort, err, 26);   // the values
                if (!ok)
                    break;
                tc_fence_after();
                uint64_t dv = smem_desc_sw128(smem_u32(kv_s + sv * Cfg::UNIT), BLK_BYTES, 1024);
                uint64_t dp = smem_desc_sw128(smem_u32(p_s + t * Cfg::P_TILE), 16, 1024);
#pragma unroll
                for (int kk = 0; kk < AT_KEYS / 16; kk++) {
                    uint64_t p_off = (uint64_t)(((kk / 4) * BLK_BYTES + (kk % 4) * 32) >> 4);
                    tc_mma(tmem + 2 * AT_KEYS + t * HD, dp + p_off, dv + (uint64_t)(kk * 128),
                           idesc_pv, (it | kk) != 0);
                }
                tc_commit(bar(11 + t));
                if (t == tiles - 1)
                    tc_commit(bar(4 + sv));        // the values' unit is free
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ row threads
        int t = (warp - 2) >> 2;                // block A or B
        int qw = warp & 3;                      // the TMEM lanes this warp may read
        int r = qw * 32 + lane;                 // this thread's row of the block
        int j = r / G, g = r - j * G;           // position within the block, head of the group
        int jq = t * R + j;                     // position within the CTA's run
        bool live = j < R && jq < q_count;
        bool tile_live = t == 0 || has_b;
        int pos = q_pos + jq;
        int lo = window > 0 && pos + 1 > window ? pos + 1 - window : 0;
        // the block's first and last position: chunks between them need no mask
        int pos_first = q_pos + t * R;
        int pos_last = min(q_pos + q_count, pos_first + R) - 1;
        int lo_last = window > 0 && pos_last + 1 > window ? pos_last + 1 - window : 0;
        uint32_t lane_addr = (uint32_t)(qw * 32) << 16;
        uint32_t tmem_s = tmem + t * AT_KEYS + lane_addr;
        uint32_t tmem_o = tmem + 2 * AT_KEYS + t * HD + lane_addr;
        const float c2 = scale * 1.4426950408889634f;      // scores in units of log2(e)
        float m_ref = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (int it = 0; it < n_chunks && tile_live; it++) {
            int t0 = (c_first + it) * AT_KEYS;              // the chunk's first key
            ok = ok && mbar_wait(bar(7 + t), it & 1, abort, err, 27);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            uint32_t raw[AT_KEYS];
            float mx = -INFINITY;
            if (ok) {
#pragma unroll
                for (int cb = 0; cb < AT_KEYS / 32; cb++)
                    tc_ld32_nowait(tmem_s + cb * 32, raw + cb * 32);
                tc_ld_wait();
                // the scores are in registers: the tensor core may write the next chunk's
                tc_fence_before();
                mbar_arrive(bar(13 + t));
                // most chunks lie wholly inside every row's range: no key is masked.
                // The maximum is taken over the raw scores (the scale is positive)
                // and scaled once; the scale itself goes into the exponent's FMA.
                bool inside = t0 + AT_KEYS - 1 <= pos_first && t0 >= lo_last;
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                if (inside && live) {
#pragma unroll
                    for (int i = 0; i < AT_KEYS; i += 4)
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            m4[e] = fmaxf(m4[e], __uint_as_float(raw[i + e]));
                } else {
#pragma unroll
                    for (int i = 0; i < AT_KEYS; i += 4)
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            int key = t0 + i + e;
                            float v = (live && key <= pos && key >= lo)
                                          ? __uint_as_float(raw[i + e]) : -INFINITY;
                            raw[i + e] = __float_as_uint(v);
                            m4[e] = fmaxf(m4[e], v);
                        }
                }
                mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * c2;
            }
            // move the row's reference only when the maximum has run far ahead of it
            bool move = mx > m_ref + PF_LAZY || (m_ref == -INFINITY && mx > -INFINITY);
            float alpha = 1.0f;
            if (move) {
                alpha = m_ref == -INFINITY ? 0.0f : exp2f(m_ref - mx);
                m_ref = mx;
                l_run *= alpha;
            }
            // with nothing visible yet the reference is -inf: subtract 0 instead, every
            // score is -inf and every weight 0
            float m_use = m_ref == -INFINITY ? 0.0f : m_ref;
            // the weights, two bfloat16 to a register, in place of the scores
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int i = 0; i < AT_KEYS / 2; i += 4) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float p0 = fast_exp2(fmaf(__uint_as_float(raw[2 * (i + e)]), c2, -m_use));
                    float p1 = fast_exp2(fmaf(__uint_as_float(raw[2 * (i + e) + 1]), c2, -m_use));
                    l4[e] += p0 + p1;
                    __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                    raw[i + e] = *reinterpret_cast<uint32_t *>(&pk);
                }
            }
            // P of the chunk before has been read, and O is whole, once that chunk's
            // P V is done: only now is that needed
            if (it > 0) {
                ok = ok && mbar_wait(bar(11 + t), (it - 1) & 1, abort, err, 28);
                ok = __all_sync(0xffffffffu, ok);
                tc_fence_after();
            }
            if (ok && it > 0 && __any_sync(0xffffffffu, move)) {
                // the warp's rows of O, 32 values at a time; rows that stay keep factor 1
#pragma unroll 1
                for (int db = 0; db < HD / 32; db++) {
                    uint32_t ov[32];
                    tc_ld32_nowait(tmem_o + db * 32, ov);
                    tc_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
                    tc_st32(tmem_o + db * 32, ov);
                }
                tc_st_wait();
            }
            if (ok) {
                uint8_t *tile = p_s + t * Cfg::P_TILE;
                // keys 8 q8 .. 8 q8 + 7: block q8 / 8, 16-byte chunk q8 % 8 of the row
#pragma unroll
                for (int q8 = 0; q8 < AT_KEYS / 8; q8++)
                    *reinterpret_cast<uint4 *>(tile + (q8 / 8) * BLK_BYTES + swz(r, q8 % 8)) =
                        make_uint4(raw[4 * q8], raw[4 * q8 + 1], raw[4 * q8 + 2], raw[4 * q8 + 3]);
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(bar(9 + t));
            l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        }
        if (tile_live) {
            ok = ok && mbar_wait(bar(11 + t), (n_chunks - 1) & 1, abort, err, 29);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            float inv = 1.0f / l_run;
            bf16 *dst = out + ((size_t)(q_row + jq) * nh + kvh * G + g) * HD;
#pragma unroll 1
            for (int db = 0; db < HD / 32; db++) {
                float ov[32];
                if (ok)
                    tc_ld32(tmem_o + db * 32, ov);
                if (ok && live) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            __nv_bfloat162 pk = __floats2bfloat162_rn(ov[i + 2 * e] * inv,
                                                                      ov[i + 2 * e + 1] * inv);
                            w[e] = *reinterpret_cast<uint32_t *>(&pk);
                        }
                        *reinterpret_cast<uint4 *>(dst + db * 32 + i) =
                            make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem), "r"((uint32_t)Cfg::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------- decode rows
// One decoded token (G <= 16 query heads of one KV head) against chunks of 128
// keys, with the keys as the M operand so that all 128 row threads have work:
//
//   S^T[key, head] = K Q^T     M = 128 keys, N = 16 (the group's heads, padded)
//   softmax over the keys      one thread per key; the maximum and the sum go
//                              through warp shuffles and shared memory
//   O^T[value, head] = V^T P   M = 128 values (V MN-major as it lies), N = 16
//
// A CTA runs over its chunks with a running (m, l, O) and leaves one partial per
// head in scratch; attention.cu's merge kernel joins the CTAs' partials.
constexpr int DQ_N = 16;                 // heads per MMA (N)
constexpr int DQ_BLK = DQ_N * 128;       // a block of 16 rows of 128 bytes
// The ring holds units of 32 KB: the keys of a chunk, then its values, then the
// next chunk's keys ...; three units, so that two CTAs fit an SM and one's waits
// are filled by the other's work.
constexpr int DQ_UNITS = 3;
constexpr int DQ_UNIT = 2 * BLK_BYTES;       // K (or V) of one chunk, 128 values each
constexpr int DQ_SMEM = 2 * DQ_BLK + 4 * DQ_BLK + DQ_UNITS * DQ_UNIT + 1024 + 1024;

// What the kernel needs to make q, and the new position's key and value, itself
// from the q,k,v product's partial sums (qkv != nullptr): then no kernel stands
// between that product and the attention.  Row r of qkv holds the heads of q, then
// of k, then of v, as float sums to be added in the order 0 .. S-1.
struct DecodeQkv {
    const float *qkv;            // nullptr: q is read through map_q and the cache is complete
    int S;
    long long split_stride;
    const void *q_w, *k_w;       // per-head RMSNorm weights of HD values, or nullptr
    int w_f32;                   // the weights are float (else bfloat16)
    float eps;
    const float *cs, *sn;        // rotation tables [positions][HD / 2], or nullptr
    bf16 *k_cache, *v_cache;     // where the new key and value go, or nullptr (a layer that
                                 // reads another layer's cache)
};

__device__ __forceinline__ float4 load_w4(const void *w, int w_f32, int at)
{
    return w_f32 ? load4((const float *)w + at) : load4((const bf16 *)w + at);
}

// GP: the group's heads rounded up to a power of two (the row threads' loops).
template <int GP>
__global__ void __launch_bounds__(192)
attn_tc_decode_kernel(const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v,
                      const int32_t *__restrict__ row_pos, const int32_t *__restrict__ row_seq,
                      const int32_t *__restrict__ block_table, int bt_stride,
                      float *__restrict__ part, int nh, int nkv, int G, int window, float scale,
                      int max_chunks, int chunks_per_cta, int row0, const DecodeQkv f)
{
    constexpr int HD = 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *q_s = smem;                       // 2 blocks of [16 heads][64 values]
    uint8_t *p_s = q_s + 2 * DQ_BLK;           // 2 buffers of 2 blocks of [16 heads][64 keys]
    uint8_t *kv_s = p_s + 4 * DQ_BLK;
    uint64_t *bars = (uint64_t *)(kv_s + DQ_UNITS * DQ_UNIT);
    // bars: 0 q_full | 1..3 unit full | 4..6 unit free | 7,8 s_full | 9,10 p_full | 11 o_full |
    //       12 pv_free | 13 the new key and value are in the cache
    uint32_t *tmem_slot = (uint32_t *)(bars + 14);
    volatile int *abort = (volatile int *)(tmem_slot + 1);
    float *red_m = (float *)(tmem_slot + 4);   // [4 warps][16 heads]
    float *red_l = red_m + 4 * DQ_N;

    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensor_map(&map_k);
        prefetch_tensor_map(&map_v);
        prefetch_tensor_map(&map_q);
    }
    int kvh = blockIdx.y;
    int parts = (max_chunks + chunks_per_cta - 1) / chunks_per_cta;
    int max_parts = parts;             // partials per (row, head) in scratch
    int lrow = blockIdx.x / parts, part_i = blockIdx.x % parts;
    int q_row = row0 + lrow;
    int q_pos = row_pos[q_row];
    int seq = row_seq[q_row];
    int lo = window > 0 && q_pos + 1 > window ? q_pos + 1 - window : 0;
    int c_base = lo / AT_KEYS;
    int c_first = c_base + part_i * chunks_per_cta;
    int c_last = min(q_pos / AT_KEYS, c_first + chunks_per_cta - 1);
    int n_chunks = c_last - c_first + 1;
    if (n_chunks <= 0)
        return;

    uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8 * i; };
    const bool fused = f.qkv != nullptr;
    // this CTA's run holds the chunk of the new position: it appends the key and value
    const bool appends = fused && f.k_cache != nullptr && c_last == q_pos / AT_KEYS;
    if (threadIdx.x == 0) {
        mbar_init(bar(0), fused ? AT_ROWS : 1);
        for (int s = 0; s < DQ_UNITS; s++) {
            mbar_init(bar(1 + s), 1);
            mbar_init(bar(4 + s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(bar(7 + b), 1);
            mbar_init(bar(9 + b), AT_ROWS);
        }
        mbar_init(bar(11), 1);
        mbar_init(bar(12), AT_ROWS);
        mbar_init(bar(13), AT_ROWS);
        *abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(64u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem = *tmem_slot;
    uint32_t tmem_s = tmem, tmem_pv = tmem + 2 * DQ_N;    // S: two buffers of 16 columns
    int *err = &g_attn_tc_error;
    // q and the keys and values of position q_pos were written by the kernel before
    // this one; every chunk before q_pos's holds what earlier steps left, so the
    // thread that loads fetches those without waiting for that kernel
    pdl_trigger();
    bool loader = warp == 0 && lane == 0;
    // The row threads make q (and the new key and value) themselves when the product's
    // sums are given: sixteen lanes share a head, each with four values of its low half
    // and the four that pair with them in the high half, a warp two heads at a time
    // (the arrangement and the order of every sum are those of rope.cu's kernel for
    // few rows, so the two give the same bits).  Rotation and norm weights were
    // written long before the kernel before this one: fetched before the wait.
    const int at4 = 4 * (lane & 15);
    float4 co = make_float4(1.0f, 1.0f, 1.0f, 1.0f), si = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 wql = co, wqh = co, wkl = co, wkh = co;
    int new_page = 0;
    if (fused && warp >= 2) {
        if (f.cs != nullptr) {
            co = load4(f.cs + (size_t)q_pos * (HD / 2) + at4);
            si = load4(f.sn + (size_t)q_pos * (HD / 2) + at4);
        }
        if (f.q_w != nullptr) {
            wql = load_w4(f.q_w, f.w_f32, at4);
            wqh = load_w4(f.q_w, f.w_f32, HD / 2 + at4);
            wkl = load_w4(f.k_w, f.w_f32, at4);
            wkh = load_w4(f.k_w, f.w_f32, HD / 2 + at4);
        }
        if (appends)
            new_page = block_table[(size_t)seq * bt_stride + q_pos / PAGE];
    }
    // The other lanes of the loader's warp do not wait either (they touch no memory):
    // a wait in one branch of a warp holds the whole warp, the loader with it.
    if (warp != 0)
        pdl_wait();

    if (fused && warp >= 2) {
        int n_slots = G + (appends ? 2 : 0);        // q heads, then the key, then the value
        int all_slots = nh + 2 * nkv;
        const float *src_row = f.qkv + (size_t)q_row * all_slots * HD;
        for (int base = 0; base < n_slots; base += 8) {
            int slot = base + (warp - 2) * 2 + (lane >> 4);
            bool live = slot < n_slots;
            bool is_q = slot < G, is_v = slot == G + 1;
            int hs = is_q ? kvh * G + slot : is_v ? nh + nkv + kvh : nh + kvh;
            float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi = lo;
            if (live) {
                const float *src = src_row + (size_t)hs * HD + at4;
                for (int s0 = 0; s0 < f.S; s0 += 4) {
                    float4 a[4], b[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (s0 + u < f.S) {
                            a[u] = load4(src + (size_t)(s0 + u) * f.split_stride);
                            b[u] = load4(src + (size_t)(s0 + u) * f.split_stride + HD / 2);
                        }
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (s0 + u < f.S) {
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
            for (int o = 8; o > 0; o >>= 1)
                ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!live)
                continue;
            if (!is_v && f.q_w != nullptr) {
                float4 wl = is_q ? wql : wkl, wh = is_q ? wqh : wkh;
                float sc = 1.0f / sqrtf(ss / (float)HD + f.eps);
                lo.x = (lo.x * sc) * wl.x; lo.y = (lo.y * sc) * wl.y;
                lo.z = (lo.z * sc) * wl.z; lo.w = (lo.w * sc) * wl.w;
                hi.x = (hi.x * sc) * wh.x; hi.y = (hi.y * sc) * wh.y;
                hi.z = (hi.z * sc) * wh.z; hi.w = (hi.w * sc) * wh.w;
            }
            if (!is_v && f.cs != nullptr) {
                float4 a = lo, b = hi;
                lo = make_float4(a.x * co.x - b.x * si.x, a.y * co.y - b.y * si.y,
                                 a.z * co.z - b.z * si.z, a.w * co.w - b.w * si.w);
                hi = make_float4(a.x * si.x + b.x * co.x, a.y * si.y + b.y * co.y,
                                 a.z * si.z + b.z * co.z, a.w * si.w + b.w * co.w);
            }
            if (is_q) {
                // where the TMA load would have put it: block of the half, row of the
                // head, 16-byte chunk at4 / 8 of the row in the 128-byte swizzle
                uint8_t *at = q_s + swz(slot, at4 / 8) + (at4 % 8) * 2;
                store4(reinterpret_cast<bf16 *>(at), lo);
                store4(reinterpret_cast<bf16 *>(at + DQ_BLK), hi);
            } else {
                bf16 *dst = (is_v ? f.v_cache : f.k_cache) +
                            (((size_t)new_page * nkv + kvh) * PAGE + (q_pos % PAGE)) * HD;
                store4(dst + at4, lo);
                store4(dst + HD / 2 + at4, hi);
            }
        }
        fence_async_smem();              // q is read by the tensor core
        tc_fence_before();
        mbar_arrive(bar(0));
        if (appends) {
            // the key and value are read back by TMA: written, made visible to that
            // proxy, then the loader is told
            __threadfence();
            asm volatile("fence.proxy.async;" ::: "memory");
            mbar_arrive(bar(13));
        }
    }

    if (loader) {
        // ---------------------------------------------------------- TMA loads
        bool waited = false;
        auto wait_and_load_q = [&]() {
            pdl_wait();
            if (!fused) {
                mbar_expect_tx(bar(0), (uint32_t)(G * HD * 2));
                tma_load_3d(smem_u32(q_s), &map_q, bar(0), 0, kvh * G, q_row);
                tma_load_3d(smem_u32(q_s + DQ_BLK), &map_q, bar(0), 64, kvh * G, q_row);
            }
            waited = true;
        };
        bool appended = !appends;
        const int32_t *bt = block_table + (size_t)seq * bt_stride;
        uint32_t armed = 0, last_parity = 0;
        for (int u = 0; u < 2 * n_chunks; u++) {        // unit u: K (even) or V (odd) of chunk u / 2
            int s = u % DQ_UNITS;
            uint32_t ph = (u / DQ_UNITS) & 1;
            if (!waited && (u >= DQ_UNITS || c_first + u / 2 >= q_pos / AT_KEYS))
                wait_and_load_q();
            if (!appended && c_first + u / 2 >= q_pos / AT_KEYS) {
                // the chunk of the new position: its key and value come from this CTA's
                // row threads
                if (!mbar_wait(bar(13), 0, abort, err, 20))
                    break;
                appended = true;
            }
            if (!mbar_wait(bar(4 + s), ph ^ 1, abort, err, 11))
                break;
            mbar_expect_tx(bar(1 + s), DQ_UNIT);
            uint32_t dst = smem_u32(kv_s + s * DQ_UNIT);
            const CUtensorMap *map = (u & 1) ? &map_v : &map_k;
            int c = c_first + u / 2;
#pragma unroll
            for (int pg = 0; pg < 2; pg++) {
                int idx = 2 * c + pg;
                int page = idx < bt_stride ? bt[idx] : -1;
                if (page < 0)
                    page = 0;          // not there: every position of it is masked
                int y = (page * nkv + kvh) * PAGE;
#pragma unroll
                for (int b = 0; b < 2; b++)
                    tma_load_2d(dst + b * BLK_BYTES + pg * (PAGE * 128), map, bar(1 + s), b * 64, y);
            }
            armed |= 1u << s;
            last_parity = (last_parity & ~(1u << s)) | (ph << s);
        }
        if (!waited)
            wait_and_load_q();
        if (*abort) {
            volatile int never = 0;
            for (int s = 0; s < DQ_UNITS; s++)
                if (armed & (1u << s))
                    mbar_wait(bar(1 + s), (last_parity >> s) & 1, &never, err, 14);
        }
    } else if (warp == 1 && lane == 0) {
        // --------------------------------------------------------------- MMAs
        constexpr uint32_t idesc_s = instr_desc_bf16(AT_KEYS, DQ_N, false, false);
        constexpr uint32_t idesc_pv = instr_desc_bf16(HD, DQ_N, false, true);
        uint32_t q_a = smem_u32(q_s), p_a = smem_u32(p_s);
        // S^T of chunk `it` into S buffer it % 2
        auto issue_s = [&](int it) -> bool {
            int u = 2 * it, s = u % DQ_UNITS;
            if (!mbar_wait(bar(1 + s), (u / DQ_UNITS) & 1, abort, err, 13))
                return false;
            tc_fence_after();
            uint32_t k_a = smem_u32(kv_s + s * DQ_UNIT);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++)
                tc_mma(tmem_s + (it & 1) * DQ_N,
                       smem_desc_sw128(k_a + (kk / 4) * BLK_BYTES + (kk % 4) * 32, 16, 1024),
                       smem_desc_sw128(q_a + (kk / 4) * DQ_BLK + (kk % 4) * 32, 16, 1024),
                       idesc_s, kk != 0);
            tc_commit(bar(7 + (it & 1)));
            tc_commit(bar(4 + s));              // the keys' unit is free once these are done
            return true;
        };
        bool ok = mbar_wait(bar(0), 0, abort, err, 12) && issue_s(0);
        for (int it = 0; it < n_chunks && ok; it++) {
            // the next chunk's scores are computed while the row threads work on this
            // one's; its S buffer was read out before P of chunk it - 1 was ready
            if (it + 1 < n_chunks)
                ok = issue_s(it + 1);
            ok = ok && mbar_wait(bar(9 + (it & 1)), (it >> 1) & 1, abort, err, 15);   // P is there
            if (ok && it > 0)
                ok = mbar_wait(bar(12), (it - 1) & 1, abort, err, 16);   // the last O^T was read
            if (!ok)
                break;
            tc_fence_after();
            int u = 2 * it + 1, s = u % DQ_UNITS;
            ok = mbar_wait(bar(1 + s), (u / DQ_UNITS) & 1, abort, err, 19);   // the values are there
            if (!ok)
                break;
            tc_fence_after();
            uint32_t v_a = smem_u32(kv_s + s * DQ_UNIT);
            uint32_t pb = p_a + (it & 1) * 2 * DQ_BLK;
#pragma unroll
            for (int kk = 0; kk < AT_KEYS / 16; kk++)
                tc_mma(tmem_pv, smem_desc_sw128(v_a + kk * 16 * 128, BLK_BYTES, 1024),
                       smem_desc_sw128(pb + (kk / 4) * DQ_BLK + (kk % 4) * 32, 16, 1024),
                       idesc_pv, kk != 0);
            tc_commit(bar(11));
            tc_commit(bar(4 + s));
        }
    } else if (warp >= 2) {
        // ---------------------------------------------- key threads / value threads
        int qw = warp & 3;
        int r = qw * 32 + lane;                 // this thread's key of the chunk, then its value
        uint32_t lane_addr = (uint32_t)(qw * 32) << 16;
        const float c2 = scale * 1.4426950408889634f;
        bool ok = true;
        // running over this CTA's chunks: maximum, sum (every thread keeps all heads')
        // and this thread's value of O for every head
        float m_run[GP], l_run[GP], o_acc[GP], alpha[GP];
#pragma unroll
        for (int g = 0; g < GP; g++) {
            m_run[g] = -INFINITY;
            l_run[g] = 0.0f;
            o_acc[g] = 0.0f;
            alpha[g] = 0.0f;
        }
        // O^T of chunk `it` joins the running O (scaled by that chunk's alpha)
        auto take_o = [&](int it) {
            ok = ok && mbar_wait(bar(11), it & 1, abort, err, 18);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            if (ok) {
                float ov[DQ_N];
                tc_ld16(tmem_pv + lane_addr, ov);
#pragma unroll
                for (int g = 0; g < GP; g++)
                    o_acc[g] = o_acc[g] * alpha[g] + ov[g];
            }
            tc_fence_before();
            mbar_arrive(bar(12));
        };
        for (int it = 0; it < n_chunks; it++) {
            int c = c_first + it;
            int t = c * AT_KEYS + r;
            bool visible = t <= q_pos && t >= lo;
            ok = ok && mbar_wait(bar(7 + (it & 1)), (it >> 1) & 1, abort, err, 17);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            float sc[DQ_N], m[GP], l[GP];
            if (ok)
                tc_ld16(tmem_s + (it & 1) * DQ_N + lane_addr, sc);
#pragma unroll
            for (int g = 0; g < GP; g++) {
                float v = (ok && visible && g < G) ? sc[g] * c2 : -INFINITY;
                sc[g] = v;
                m[g] = warp_max(v);
            }
            if (lane == 0) {
#pragma unroll
                for (int g = 0; g < GP; g++)
                    red_m[qw * DQ_N + g] = m[g];
            }
            named_barrier(1, AT_ROWS);
            // the chunk before this one is taken into O with ITS alpha, before alpha
            // is overwritten below
            if (it > 0)
                take_o(it - 1);
#pragma unroll
            for (int g = 0; g < GP; g++) {
                float mc = fmaxf(fmaxf(red_m[g], red_m[DQ_N + g]),
                                 fmaxf(red_m[2 * DQ_N + g], red_m[3 * DQ_N + g]));
                float mn = fmaxf(m_run[g], mc);
                alpha[g] = m_run[g] == -INFINITY ? 0.0f : exp2f(m_run[g] - mn);
                if (mn == -INFINITY)
                    alpha[g] = 1.0f;
                m_run[g] = mn;
                float p = sc[g] == -INFINITY ? 0.0f : exp2f(sc[g] - mn);
                sc[g] = p;
                l[g] = warp_sum(p);
            }
            if (lane == 0) {
#pragma unroll
                for (int g = 0; g < GP; g++)
                    red_l[qw * DQ_N + g] = l[g];
            }
            // P[head][key] in bfloat16, buffer it % 2 (chunk it - 2's P V has been waited
            // for): block r / 64, row g, 16-byte chunk (r % 64) / 8
            {
                uint8_t *blk = p_s + (it & 1) * 2 * DQ_BLK + (r / 64) * DQ_BLK;
                int j = (r % 64) / 8, e = (r % 8) * 2;
#pragma unroll
                for (int g = 0; g < GP; g++)
                    if (g < G)
                        *reinterpret_cast<bf16 *>(blk + swz(g, j) + e) = __float2bfloat16_rn(sc[g]);
            }
            fence_async_smem();
            named_barrier(1, AT_ROWS);
            tc_fence_before();
            mbar_arrive(bar(9 + (it & 1)));
#pragma unroll
            for (int g = 0; g < GP; g++)
                l_run[g] = l_run[g] * alpha[g] + (red_l[g] + red_l[DQ_N + g] + red_l[2 * DQ_N + g] +
                                                  red_l[3 * DQ_N + g]);
        }
        take_o(n_chunks - 1);
        // one partial for this CTA's run of chunks
        if (ok) {
            int pi = part_i;
#pragma unroll
            for (int g = 0; g < GP; g++) {
                if (g >= G)
                    continue;
                float *dst = part + (((size_t)lrow * nh + kvh * G + g) * max_parts + pi) *
                                        (size_t)(HD + 2);
                if (r == g) {
                    dst[0] = m_run[g] * 0.6931471805599453f;   // the merge works in natural logs
                    dst[1] = l_run[g];
                }
                dst[2 + r] = o_acc[g];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                     ::"r"(tmem), "r"(64u) : "memory");
    }
}

// ------------------------------------------------------------------ host side
struct MapKey {
    const void *ptr;
    long long d0, d1, d2;
    int b0, b1, b2;
    bool operator<(const MapKey &o) const
    {
        return std::tie(ptr, d0, d1, d2, b0, b1, b2) <
               std::tie(o.ptr, o.d0, o.d1, o.d2, o.b0, o.b1, o.b2);
    }
};

// A bfloat16 tensor of rank 2 or 3 (dims innermost first, d2 = 0 for rank 2),
// dense, read in boxes of (64, b1[, b2]) with the 128-byte swizzle.
static bool attn_tensor_map(const void *ptr, long long d0, long long d1, long long d2, int b1,
                            int b2, CUtensorMap *out)
{
    static std::map<MapKey, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{ptr, d0, d1, d2, 64, b1, b2};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiled enc = tensor_map_encoder();
    if (!enc)
        return false;
    int rank = d2 > 0 ? 3 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)(d2 > 0 ? d2 : 1)};
    cuuint64_t strides[2] = {(cuuint64_t)d0 * 2, (cuuint64_t)d0 * d1 * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)b1, (cuuint32_t)(b2 > 0 ? b2 : 1)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap map;
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(ptr), dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 8192)
        cache.clear();
    cache[key] = map;
    *out = map;
    return true;
}

template <int HD>
static int launch_attn_rows(const void *q, const void *k_cache, const void *v_cache,
                            long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                            const int32_t *block_table, int bt_stride, float *part, int n, int nh,
                            int nkv, int window, float scale, int max_chunks, int chunks_per_cta,
                            int row0, int n_rows, cudaStream_t st)
{
    using Cfg = AttnCfg<HD>;
    int G = nh / nkv;
    CUtensorMap mq, mk, mv;
    if (!attn_tensor_map(q, HD, nh, n, G, 1, &mq) ||
        !attn_tensor_map(k_cache, HD, n_pages * nkv * PAGE, 0, PAGE, 0, &mk) ||
        !attn_tensor_map(v_cache, HD, n_pages * nkv * PAGE, 0, PAGE, 0, &mv))
        return JB_EINVAL;
    auto kern = attn_tc_rows_kernel<HD>;
    static unsigned long long smem_allowed = 0;
    if (!allow_dynamic_smem(kern, Cfg::SMEM_BYTES, smem_allowed))
        return JB_ELAUNCH;
    unsigned gx = (unsigned)n_rows * ((max_chunks + chunks_per_cta - 1) / chunks_per_cta);
    if (gx == 0)
        return JB_OK;
    launch(kern, dim3(gx, nkv), 192, Cfg::SMEM_BYTES, st, mq, mk, mv, row_pos, row_seq,
           block_table, bt_stride, part, nh, nkv, G, window, scale, max_chunks, chunks_per_cta,
           row0);
    return launch_status();
}

}  // namespace jb

using namespace jb;

// Whether the tensor-core attention takes these sizes: heads of 64 or 128
// values, at most 128 query heads per KV head.
extern "C" int jb_attn_tc_ok(int nh, int nkv, int hd)
{
    return nkv > 0 && nh % nkv == 0 && nh / nkv <= AT_ROWS && (hd == 64 || hd == 128) &&
           nkv <= 65535;
}

// Positions of one sequence that a CTA of the prefill kernel holds (an entry of qblk).
extern "C" int jb_attn_tc_block_positions(int nh, int nkv)
{
    int G = nh / nkv;
    return 2 * (AT_ROWS / G);      // a CTA of the prefill kernel holds two blocks of 128 rows
}

// Prefill rows.  q, out: [n, nh, hd] bfloat16; caches [n_pages, nkv, PAGE, hd].
// qblk: int32 [n_blocks][4] = first row, positions (<= block positions), the
// first row's position, the sequence's index in block_table; CTAs start in this
// order, so the runs that see the most keys should come first.
extern "C" int jb_attn_tc_prefill(const void *q, const void *k_cache, const void *v_cache,
                                  long long n_pages, const int32_t *qblk, int n_blocks,
                                  const int32_t *block_table, int bt_stride, void *out, int n,
                                  int nh, int nkv, int hd, int window, float scale, cudaStream_t st)
{
    if (!jb_attn_tc_ok(nh, nkv, hd) || n <= 0)
        return JB_EINVAL;
    int G = nh / nkv;
    int R = AT_ROWS / G;               // positions of one block; qblk's runs hold up to 2 R
    CUtensorMap mq, mk, mv;
    if (!attn_tensor_map(q, hd, nh, n, G, R, &mq) ||
        !attn_tensor_map(k_cache, hd, n_pages * nkv * PAGE, 0, PAGE, 0, &mk) ||
        !attn_tensor_map(v_cache, hd, n_pages * nkv * PAGE, 0, PAGE, 0, &mv))
        return JB_EINVAL;
    if (n_blocks <= 0)
        return JB_OK;
#define JB_PF(HDV)                                                                             \
    do {                                                                                       \
        static unsigned long long smem_allowed = 0;                                            \
        if (!allow_dynamic_smem(attn_tc_prefill_kernel<HDV>, PrefillCfg<HDV>::SMEM_BYTES,      \
                                smem_allowed))                                                 \
            return JB_ELAUNCH;                                                                 \
        launch(attn_tc_prefill_kernel<HDV>, dim3((unsigned)n_blocks * nkv), PF_THREADS,        \
               PrefillCfg<HDV>::SMEM_BYTES, st, mq, mk, mv, qblk, block_table, bt_stride,      \
               (bf16 *)out, nh, nkv, G, R, window, scale);                                     \
    } while (0)
    if (hd == 128)
        JB_PF(128);
    else
        JB_PF(64);
#undef JB_PF
    return launch_status();
}

// Decode rows row0 .. row0 + n_rows - 1 (one token each): writes the per-chunk
// partials of attention.cu's layout into `part`; jb_attention_merge joins them.
static int attn_tc_decode(const void *q, const void *k_cache, const void *v_cache,
                          long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                          const int32_t *block_table, int bt_stride, float *part, int n,
                          int row0, int n_rows, int nh, int nkv, int hd, int window,
                          float scale, int max_chunks, int chunks_per_cta, const DecodeQkv &f,
                          cudaStream_t st)
{
    if (!jb_attn_tc_ok(nh, nkv, hd) || n_rows <= 0 || max_chunks <= 0 || chunks_per_cta <= 0)
        return JB_EINVAL;
    if (f.qkv != nullptr && !(hd == 128 && nh / nkv <= DQ_N))
        return JB_EINVAL;
    if (hd == 128 && nh / nkv <= DQ_N) {
        int G = nh / nkv;
        CUtensorMap mq, mk, mv;
        if (!attn_tensor_map(k_cache, hd, n_pages * nkv * PAGE, 0, PAGE, 0, &mk) ||
            !attn_tensor_map(v_cache, hd, n_pages * nkv * PAGE, 0, PAGE, 0, &mv))
            return JB_EINVAL;
        if (f.qkv != nullptr)
            mq = mk;            // not used: the kernel makes q itself
        else if (!attn_tensor_map(q, hd, nh, n, G, 1, &mq))
            return JB_EINVAL;
        unsigned gx = (unsigned)n_rows * ((max_chunks + chunks_per_cta - 1) / chunks_per_cta);
#define JB_DQ(GP)                                                                              \
    do {                                                                                       \
        static unsigned long long smem_allowed = 0;                                            \
        if (!allow_dynamic_smem(attn_tc_decode_kernel<GP>, DQ_SMEM, smem_allowed))             \
            return JB_ELAUNCH;                                                                 \
        launch(attn_tc_decode_kernel<GP>, dim3(gx, nkv), 192, DQ_SMEM, st,                     \
               mq, mk, mv, row_pos, row_seq, block_table, bt_stride, part, nh, nkv, G, window, \
               scale, max_chunks, chunks_per_cta, row0, f);                                    \
    } while (0)
        if (G <= 1)
            JB_DQ(1);
        else if (G <= 2)
            JB_DQ(2);
        else if (G <= 4)
            JB_DQ(4);
        else if (G <= 8)
            JB_DQ(8);
        else
            JB_DQ(16);
#undef JB_DQ
        return launch_status();
    }
    if (hd == 128)
        return launch_attn_rows<128>(q, k_cache, v_cache, n_pages, row_pos, row_seq, block_table,
                                     bt_stride, part, n, nh, nkv, window, scale, max_chunks,
                                     chunks_per_cta, row0, n_rows, st);
    return launch_attn_rows<64>(q, k_cache, v_cache, n_pages, row_pos, row_seq, block_table,
                                bt_stride, part, n, nh, nkv, window, scale, max_chunks,
                                chunks_per_cta, row0, n_rows, st);
}

extern "C" int jb_attn_tc_decode(const void *q, const void *k_cache, const void *v_cache,
                                 long long n_pages, const int32_t *row_pos, const int32_t *row_seq,
                                 const int32_t *block_table, int bt_stride, float *part, int n,
                                 int row0, int n_rows, int nh, int nkv, int hd, int window,
                                 float scale, int max_chunks, int chunks_per_cta, cudaStream_t st)
{
    DecodeQkv f = {};
    return attn_tc_decode(q, k_cache, v_cache, n_pages, row_pos, row_seq, block_table, bt_stride,
                          part, n, row0, n_rows, nh, nkv, hd, window, scale, max_chunks,
                          chunks_per_cta, f, st);
}

// The same, with q and the new position's key and value made by the attention kernel
// itself from the q,k,v product's partial sums (see DecodeQkv): per-head RMSNorm with
// q_w / k_w (or none), rotation by cs / sn at the row's position (or none), key and
// value written to the row's place in the cache when append is set.  Heads of 128
// values in groups of up to 16 only (jb_attn_tc_decode_runs); everything 16-byte
// aligned (8 for bfloat16 weights).
extern "C" int jb_attn_tc_decode_qkv(const float *qkv, int S, long long split_stride,
                                     const void *q_w, const void *k_w, int w_dt, float eps,
                                     const float *cs, const float *sn, void *k_cache,
                                     void *v_cache, int append, long long n_pages,
                                     const int32_t *row_pos, const int32_t *row_seq,
                                     const int32_t *block_table, int bt_stride, float *part, int n,
                                     int row0, int n_rows, int nh, int nkv, int hd, int window,
                                     float scale, int max_chunks, int chunks_per_cta,
                                     cudaStream_t st)
{
    auto aligned = [](const void *p, size_t to) { return (uintptr_t)p % to == 0; };
    if (qkv == nullptr || S <= 0 || split_stride % 4 != 0 || !aligned(qkv, 16) ||
        (q_w == nullptr) != (k_w == nullptr) || (cs == nullptr) != (sn == nullptr) ||
        (w_dt != JB_F32 && w_dt != JB_BF16))
        return JB_EINVAL;
    size_t w_to = w_dt == JB_F32 ? 16 : 8;
    if (!aligned(q_w, w_to) || !aligned(k_w, w_to) || !aligned(cs, 16) || !aligned(sn, 16))
        return JB_EINVAL;
    DecodeQkv f = {qkv, S, split_stride, q_w, k_w, w_dt == JB_F32, eps, cs, sn,
                   append ? (bf16 *)k_cache : nullptr, append ? (bf16 *)v_cache : nullptr};
    return attn_tc_decode(nullptr, k_cache, v_cache, n_pages, row_pos, row_seq, block_table,
                          bt_stride, part, n, row0, n_rows, nh, nkv, hd, window, scale, max_chunks,
                          chunks_per_cta, f, st);
}

// Whether the decode kernel for these sizes runs over several chunks per CTA and
// leaves one partial per CTA (1), or wants one chunk per CTA (0).
extern "C" int jb_attn_tc_decode_runs(int nh, int nkv, int hd)
{
    return jb_attn_tc_ok(nh, nkv, hd) && hd == 128 && nh / nkv <= DQ_N;
}

extern "C" int jb_attn_tc_error(void)
{
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_tc_error, sizeof v) != cudaSuccess)
        return JB_ELAUNCH;
    if (v != 0)
        cudaMemcpyToSymbol(g_attn_tc_error, &zero, sizeof zero);
    return v;
}
