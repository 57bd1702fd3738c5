// Choosing a token from a row of logits on the device: the first maximum, or
// a draw after temperature, top-k, top-p and min-p.
//
// The draw follows the reference's sampler step by step
// (src/llm/sample.c:283-342): the candidates are the logits not below
// max - 30 T; with 0 < top_k < vocab only the top_k largest of them (equal
// logits: the lower id first); sorted by falling logit, then rising id;
// p_i = exp((l_i - l_0) / T) summed in double in that order; top_p keeps the
// shortest prefix whose mass reaches top_p * sum; min_p drops what lies below
// min_p * p_0; one splitmix64 number (src/llm/sample.c:133-139), scaled by the
// sum, picks by walking the prefix.  A row with T <= 0 takes the first index
// of the maximum (src/llm/sample.c:141-148) and uses no random number.
//
// Two kernels on the usual way.  The first cuts every row into chunks of CHUNK
// logits and lets a block find each chunk's CHUNK_KEEP best, in order (value
// falling, id rising; with ids in the keys that is exact).  The second has one
// block per row: it merges the chunks' lists, which hold the row's CHUNK_KEEP
// best, and draws.  A row that wants more candidates than that (top_k off or
// above CHUNK_KEEP) goes the long way, for which the caller gives scratch: every
// logit not below the floor becomes a key, all SMs sort the keys (a bitonic
// network: blocks sort 4,096 keys in shared memory, steps across blocks run as
// kernels of their own), and the row's block walks the sorted candidates with
// prefix sums in place of the reference's one thread.
#include "common.cuh"
#include "kernels.h"

namespace jb {

constexpr int SAMPLE_THREADS = 1024;
constexpr int CHUNK = 4096;          // logits a block of the first kernel sorts
constexpr int CHUNK_KEEP = 64;       // candidates it keeps
constexpr int MERGE_CAP = 4096;      // candidates of all chunks of a row that the second kernel merges
constexpr int SORT_BLOCK = 4096;     // keys a block of the long way's sort holds in shared memory

__device__ __forceinline__ uint32_t ordered_key(float f)
{
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_value(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t *state)
{
    uint64_t z = (*state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// Ascending bitonic sort of n = a power of two keys, by the whole block.
__device__ void bitonic_sort(uint64_t *keys, int n)
{
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
                int lo = 2 * i - (i & (stride - 1));
                int hi = lo + stride;
                bool up = (lo & size) == 0;
                uint64_t a = keys[lo], b = keys[hi];
                if ((a > b) == up) {
                    keys[lo] = b;
                    keys[hi] = a;
                }
            }
        }
    }
    __syncthreads();
}

// The draw among nc candidates in their order (falling probability), by one
// thread: top_p keeps the shortest prefix whose mass reaches top_p * sum, min_p
// drops what lies below min_p * p_0, one splitmix64 number picks by walking.
__device__ void draw(const uint64_t *keys, const float *probs, unsigned nc, float tp, float mp,
                     uint64_t *rng_state, int32_t *out, int32_t *forced)
{
    double sum = 0.0;
    for (unsigned i = 0; i < nc; i++)
        sum += (double)probs[i];
    if (tp > 0.0f && tp < 1.0f) {
        double c = 0.0;
        double lim = (double)tp * sum;
        unsigned kk = 0;
        while (kk < nc && c < lim)
            c += (double)probs[kk++];
        nc = kk;
        sum = c;
    }
    if (mp > 0.0f) {
        unsigned kk = 1;
        float lim = mp * probs[0];
        while (kk < nc && probs[kk] >= lim)
            kk++;
        for (unsigned i = kk; i < nc; i++)
            sum -= (double)probs[i];
        nc = kk;
    }
    if (forced)
        *forced = nc <= 1;
    uint64_t state = *rng_state;
    double u = (double)(splitmix64(&state) >> 11) * 0x1.0p-53 * sum;
    *rng_state = state;
    int32_t pick = (int32_t)(uint32_t)keys[nc - 1];
    for (unsigned i = 0; i + 1 < nc; i++) {
        u -= (double)probs[i];
        if (u < 0) {
            pick = (int32_t)(uint32_t)keys[i];
            break;
        }
    }
    *out = pick;
}


// keys of a candidate: the logit's order-preserving bits inverted in the upper
// half, its id in the lower, so that ascending keys are falling logits and, among
// equal logits, rising ids
__device__ __forceinline__ uint64_t candidate_key(float v, int id)
{
    return ((uint64_t)(~ordered_key(v)) << 32) | (uint32_t)id;
}

// Ascending sort of the 128 keys of a warp, four per lane: key j of lane l is
// element 4 l + j.  A bitonic network; steps between lanes go through shuffles.
__device__ __forceinline__ void warp_sort128(uint64_t (&k)[4], int lane)
{
#pragma unroll
    for (int size = 2; size <= 128; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 4) {
                bool lower = (lane & (stride >> 2)) == 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint64_t other = __shfl_xor_sync(0xffffffffu, k[j], stride >> 2);
                    bool up = (((lane << 2) | j) & size) == 0;
                    k[j] = (lower == up) ? min(k[j], other) : max(k[j], other);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if ((j & stride) == 0) {
                        bool up = (((lane << 2) | j) & size) == 0;
                        uint64_t a = k[j], c = k[j | stride];
                        k[j] = up ? min(a, c) : max(a, c);
                        k[j | stride] = up ? max(a, c) : min(a, c);
                    }
                }
            }
        }
    }
}

// Ascending sort of a bitonic sequence of 64 keys, two per lane (element 2 l + j).
__device__ __forceinline__ void warp_merge64(uint64_t (&v)[2], int lane)
{
#pragma unroll
    for (int stride = 32; stride >= 2; stride >>= 1) {
        bool lower = (lane & (stride >> 1)) == 0;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            uint64_t other = __shfl_xor_sync(0xffffffffu, v[j], stride >> 1);
            v[j] = lower ? min(v[j], other) : max(v[j], other);
        }
    }
    uint64_t a = v[0], c = v[1];
    v[0] = min(a, c);
    v[1] = max(a, c);
}

// Block (row, chunk): the chunk's CHUNK_KEEP best candidates, in order, into
// chunk_keys[row][chunk][CHUNK_KEEP] (first_only: only the best one).  Every warp
// sorts its 128 keys in registers and keeps the best 64; the warps' lists are then
// merged two by two, each time keeping the best 64 of 128, until one is left.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_chunks_kernel(const float *__restrict__ logits, int V, int chunks,
                     uint64_t *__restrict__ chunk_keys, int first_only)
{
    static_assert(CHUNK == 4 * SAMPLE_THREADS && CHUNK_KEEP == 64, "the merge below is for these");
    __shared__ uint64_t lists[2][SAMPLE_THREADS / 32][CHUNK_KEEP];
    pdl_trigger();
    pdl_wait();
    int row = blockIdx.x / chunks, c = blockIdx.x % chunks, tid = threadIdx.x;
    int lane = tid & 31, warp = tid >> 5;
    const float *lg = logits + (size_t)row * V;
    uint64_t *dst = chunk_keys + ((size_t)row * chunks + c) * CHUNK_KEEP;
    uint64_t mine[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        int i = c * CHUNK + tid + j * SAMPLE_THREADS;
        mine[j] = i < V ? candidate_key(lg[i], i) : ~0ull;
    }
    if (first_only) {
        uint64_t best = min(min(mine[0], mine[1]), min(mine[2], mine[3]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
        if (lane == 0)
            lists[0][0][warp] = best;
        __syncthreads();
        if (warp == 0) {
            best = lists[0][0][lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
            if (lane == 0)
                dst[0] = best;
        }
        return;
    }
    warp_sort128(mine, lane);
    if (lane < 16) {                            // elements 0 .. 63: the warp's best
#pragma unroll
        for (int j = 0; j < 4; j++)
            lists[0][warp][4 * lane + j] = mine[j];
    }
    __syncthreads();
    int buf = 0;
    for (int n = SAMPLE_THREADS / 32; n > 1; n >>= 1, buf ^= 1) {
        if (warp < n / 2) {
            // A rising, B falling: a bitonic sequence whose lower half after one
            // compare step holds the best 64 of the 128
            uint64_t v[2];
#pragma unroll
            for (int j = 0; j < 2; j++) {
                int i = 2 * lane + j;
                v[j] = min(lists[buf][2 * warp][i], lists[buf][2 * warp + 1][CHUNK_KEEP - 1 - i]);
            }
            warp_merge64(v, lane);
            lists[buf ^ 1][warp][2 * lane] = v[0];
            lists[buf ^ 1][warp][2 * lane + 1] = v[1];
        }
        __syncthreads();
    }
    if (tid < CHUNK_KEEP)
        dst[tid] = lists[buf][0][tid];
}

// ------------------------------------------------------------- the long way
// The least key among the chunks' best: the row's first maximum.
__device__ __forceinline__ uint64_t row_best(const uint64_t *chunk_keys, int row, int chunks,
                                             uint64_t *shared32)
{
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint64_t *src = chunk_keys + (size_t)row * chunks * CHUNK_KEEP;
    uint64_t best = ~0ull;
    for (int c = tid; c < chunks; c += blockDim.x)
        best = min(best, src[(size_t)c * CHUNK_KEEP]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (lane == 0)
        shared32[warp] = best;
    __syncthreads();
    best = shared32[lane < (int)(blockDim.x >> 5) ? lane : 0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
    __syncthreads();
    return best;
}

// keys[row][i], i < P: the candidate key of logit i when it is not below the
// row's floor (max - 30 T), else the key that sorts last.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_fill_kernel(const float *__restrict__ logits, int V, const int32_t *__restrict__ row_slot,
                   const float *__restrict__ temperature, const uint64_t *__restrict__ chunk_keys,
                   int chunks, uint64_t *__restrict__ keys, long long P)
{
    __shared__ uint64_t shared32[32];
    pdl_trigger();
    pdl_wait();
    int row = blockIdx.y;
    long long i = (long long)blockIdx.x * SAMPLE_THREADS + threadIdx.x;
    int slot = row_slot ? row_slot[row] : row;
    float T = temperature[slot];
    float top = key_value(~(uint32_t)(row_best(chunk_keys, row, chunks, shared32) >> 32));
    float floor_v = top - 30.0f * T;
    if (i >= P)
        return;
    uint64_t key = ~0ull;
    if (T > 0.0f && i < V) {
        float v = logits[(size_t)row * V + i];
        if (v >= floor_v)
            key = candidate_key(v, (int)i);
    }
    keys[(size_t)row * P + i] = key;
}

// One compare step of the bitonic network on keys in shared memory; idx0 is the
// global index of the block's first key (it decides the direction).
__device__ __forceinline__ void sort_step_shared(uint64_t *k, long long idx0, long long size,
                                                 int stride)
{
    for (int t = threadIdx.x; t < SORT_BLOCK / 2; t += blockDim.x) {
        int lo = 2 * t - (t & (stride - 1));
        int hi = lo + stride;
        bool up = ((idx0 + lo) & size) == 0;
        uint64_t a = k[lo], b = k[hi];
        if ((a > b) == up) {
            k[lo] = b;
            k[hi] = a;
        }
    }
    __syncthreads();
}

// A block's SORT_BLOCK keys of one row: FULL: sorted from scratch (every size up to
// SORT_BLOCK); else the steps of `size` whose partners lie inside the block.
template <bool FULL>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sort_local_kernel(uint64_t *__restrict__ keys, long long P, long long size)
{
    __shared__ uint64_t k[SORT_BLOCK];
    pdl_trigger();
    pdl_wait();
    long long idx0 = (long long)blockIdx.x * SORT_BLOCK;
    uint64_t *row_keys = keys + (size_t)blockIdx.y * P + idx0;
    int n = (int)min((long long)SORT_BLOCK, P - idx0);      // P is a power of two: n too
    for (int t = threadIdx.x; t < SORT_BLOCK; t += blockDim.x)
        k[t] = t < n ? row_keys[t] : ~0ull;
    __syncthreads();
    if (FULL) {
        for (long long sz = 2; sz <= SORT_BLOCK; sz <<= 1)
            for (int st = (int)(sz >> 1); st > 0; st >>= 1)
                sort_step_shared(k, idx0, sz, st);
    } else {
        for (int st = SORT_BLOCK / 2; st > 0; st >>= 1)
            sort_step_shared(k, idx0, size, st);
    }
    for (int t = threadIdx.x; t < n; t += blockDim.x)
        row_keys[t] = k[t];
}

// One compare step whose partners lie in different blocks.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sort_global_kernel(uint64_t *__restrict__ keys, long long P, long long size, long long stride)
{
    pdl_trigger();
    pdl_wait();
    long long t = (long long)blockIdx.x * SAMPLE_THREADS + threadIdx.x;
    if (t >= P / 2)
        return;
    uint64_t *k = keys + (size_t)blockIdx.y * P;
    long long lo = 2 * t - (t & (stride - 1));
    long long hi = lo + stride;
    bool up = (lo & size) == 0;
    uint64_t a = k[lo], b = k[hi];
    if ((a > b) == up) {
        k[lo] = b;
        k[hi] = a;
    }
}

// The sum of v over the block, in double, to every thread; tmp: 32 doubles.
__device__ __forceinline__ double block_sum_double(double v, double *tmp)
{
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0)
        tmp[warp] = v;
    __syncthreads();
    double t = lane < (int)(blockDim.x >> 5) ? tmp[lane] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// The draw among n candidates in their order by the whole block: the same cuts as
// draw() above, with every thread walking a run of consecutive candidates from the
// sum of the runs before it.  (Sums of other groupings than the reference's one by
// one: they differ from it in the last bits of a double.)
__device__ void draw_parallel(const uint64_t *keys, const float *probs, unsigned n, float tp,
                              float mp, uint64_t *rng_state, int32_t *out, int32_t *forced,
                              double *tmp, unsigned *sh_idx, double *sh_val)
{
    int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned per = (n + blockDim.x - 1) / blockDim.x;
    unsigned a = min(n, tid * per), b = min(n, a + per);
    double local = 0.0;
    for (unsigned i = a; i < b; i++)
        local += (double)probs[i];
    // what lies before this thread's run: a scan over the threads' sums
    double incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o)
            incl += up;
    }
    __syncthreads();
    if (lane == 31)
        tmp[warp] = incl;
    __syncthreads();
    double before = 0.0, total = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
        double t = tmp[w];
        before += w < warp ? t : 0.0;
        total += t;
    }
    double off = before + incl - local;
    unsigned nc = n;
    double sum = total;
    __syncthreads();
    if (tp > 0.0f && tp < 1.0f) {
        // the shortest prefix whose mass reaches tp * sum (all of them if, by a last
        // bit, none does)
        const unsigned NONE = 0xffffffffu;
        double lim = (double)tp * sum;
        if (tid == 0)
            *sh_idx = NONE;
        __syncthreads();
        unsigned found = NONE;
        double c = off;
        if (off < lim) {
            for (unsigned i = a; i < b; i++) {
                c += (double)probs[i];
                if (c >= lim) {
                    found = i + 1;
                    break;
                }
            }
        }
        if (found != NONE)
            atomicMin(sh_idx, found);
        __syncthreads();
        unsigned kk = *sh_idx;
        if (kk != NONE && found == kk)
            *sh_val = c;                        // the one thread whose run holds the crossing
        __syncthreads();
        if (kk != NONE) {
            nc = kk;
            sum = *sh_val;
        }
        __syncthreads();
    }
    if (mp > 0.0f) {
        // what lies below mp * p_0 goes, and its mass with it
        float lim = mp * probs[0];
        if (tid == 0)
            *sh_idx = nc;
        __syncthreads();
        unsigned first = nc;
        for (unsigned i = max(a, 1u); i < min(b, nc); i++)
            if (probs[i] < lim) {
                first = i;
                break;
            }
        if (first < nc)
            atomicMin(sh_idx, first);
        __syncthreads();
        unsigned kk = *sh_idx;
        double gone = 0.0;
        for (unsigned i = max(a, kk); i < min(b, nc); i++)
            gone += (double)probs[i];
        gone = block_sum_double(gone, tmp);
        sum -= gone;
        nc = kk;
        __syncthreads();
    }
    if (tid == 0) {
        if (forced)
            *forced = nc <= 1;
        uint64_t state = *rng_state;
        *sh_val = (double)(splitmix64(&state) >> 11) * 0x1.0p-53 * sum;
        *rng_state = state;
        *sh_idx = nc - 1;                       // the last candidate, unless the walk ends before
    }
    __syncthreads();
    double u = *sh_val;
    {
        double c = off;
        unsigned found = n;
        if (off <= u) {
            for (unsigned i = a; i < min(b, nc - 1); i++) {
                c += (double)probs[i];
                if (c > u) {
                    found = i;
                    break;
                }
            }
        }
        if (found < n)
            atomicMin(sh_idx, found);
    }
    __syncthreads();
    if (tid == 0)
        *out = (int32_t)(uint32_t)keys[*sh_idx];
}

// ------------------------------------------------------------ a row's choice
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float *__restrict__ logits, int V, const int32_t *__restrict__ row_slot,
              const float *__restrict__ temperature, const int32_t *__restrict__ top_k,
              const float *__restrict__ top_p, const float *__restrict__ min_p,
              uint64_t *__restrict__ rng, uint64_t *__restrict__ big_keys,
              float *__restrict__ big_probs, long long big_cap,
              const uint64_t *__restrict__ chunk_keys, int chunks, int chunk_kept,
              int32_t *__restrict__ out, int32_t *__restrict__ forced)
{
    __shared__ uint64_t small_keys[MERGE_CAP];
    __shared__ float small_probs[CHUNK_KEEP];
    __shared__ double tmp[32];
    __shared__ double sh_val;
    __shared__ unsigned sh_idx, n_elig;

    pdl_trigger();
    pdl_wait();
    int row = blockIdx.x, tid = threadIdx.x;
    int lane = tid & 31, warp = tid >> 5;
    int slot = row_slot ? row_slot[row] : row;
    float T = temperature ? temperature[slot] : 0.0f;
    int tk = top_k ? top_k[slot] : 0;
    const uint64_t *src = chunk_keys + (size_t)row * chunks * CHUNK_KEEP;

    if (!(T > 0.0f)) {
        // the first maximum: the least key among the chunks' best
        uint64_t best = row_best(chunk_keys, row, chunks, small_keys);
        if (tid == 0) {
            out[row] = (int32_t)(uint32_t)best;
            if (forced)
                forced[row] = 0;
        }
        return;
    }
    if (tk > 0 && tk <= chunk_kept && chunk_kept == CHUNK_KEEP && tk < V &&
        chunks * CHUNK_KEEP <= MERGE_CAP) {
        // ---- the usual way: the chunks' lists hold all this row can want.  The
        // lists (each sorted, up to 64 of them) are merged two by two, keeping the
        // best 64 of 128 each time, in place: the warp that merges lists a and
        // a + step writes into a
        static_assert(MERGE_CAP == 64 * CHUNK_KEEP, "64 lists of CHUNK_KEEP keys");
        for (int i = tid; i < MERGE_CAP; i += SAMPLE_THREADS)
            small_keys[i] = i / CHUNK_KEEP < chunks ? src[i] : ~0ull;
        __syncthreads();
        for (int step = 1; step < 64; step <<= 1) {
            int a = 2 * step * warp;
            if (a + step < 64) {
                uint64_t v[2];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    int i = 2 * lane + j;
                    v[j] = min(small_keys[a * CHUNK_KEEP + i],
                               small_keys[(a + step) * CHUNK_KEEP + CHUNK_KEEP - 1 - i]);
                }
                warp_merge64(v, lane);
                small_keys[a * CHUNK_KEEP + 2 * lane] = v[0];
                small_keys[a * CHUNK_KEEP + 2 * lane + 1] = v[1];
            }
            __syncthreads();
        }
        // the tk best of the row, of which those not below max - 30 T count
        float top = key_value(~(uint32_t)(small_keys[0] >> 32));
        float floor_v = top - 30.0f * T;
        if (tid == 0)
            n_elig = 0;
        __syncthreads();
        if (tid < tk) {
            uint64_t k = small_keys[tid];
            float l = key_value(~(uint32_t)(k >> 32));
            bool in = k != ~0ull && l >= floor_v;
            small_probs[tid] = in ? expf((l - top) / T) : 0.0f;
            if (in)
                atomicAdd(&n_elig, 1u);      // they are a prefix: the keys are sorted
        }
        __syncthreads();
        if (tid == 0)
            draw(small_keys, small_probs, n_elig, top_p ? top_p[slot] : 0.0f,
                 min_p ? min_p[slot] : 0.0f, rng + slot, out + row, forced ? forced + row : nullptr);
        return;
    }

    // ---- the long way: the row's candidates lie sorted in the caller's scratch
    if (big_keys == nullptr || big_probs == nullptr || big_cap < V) {
        if (tid == 0)
            out[row] = -1;      // no scratch for this many candidates
        return;
    }
    const uint64_t *keys = big_keys + (size_t)row * big_cap;
    float *probs = big_probs + (size_t)row * big_cap;
    if (tid == 0) {
        // how many candidates: the first key that sorts last ends them
        long long lo = 0, hi = V;
        while (lo < hi) {
            long long mid = (lo + hi) >> 1;
            if (keys[mid] == ~0ull)
                hi = mid;
            else
                lo = mid + 1;
        }
        n_elig = (unsigned)lo;
    }
    __syncthreads();
    unsigned K = tk > 0 && tk < V ? (unsigned)tk : (unsigned)V;
    unsigned n_sel = min(n_elig, K);
    float top = key_value(~(uint32_t)(keys[0] >> 32));
    for (unsigned i = tid; i < n_sel; i += SAMPLE_THREADS)
        probs[i] = expf((key_value(~(uint32_t)(keys[i] >> 32)) - top) / T);
    __syncthreads();
    draw_parallel(keys, probs, n_sel, top_p ? top_p[slot] : 0.0f, min_p ? min_p[slot] : 0.0f,
                  rng + slot, out + row, forced ? forced + row : nullptr, tmp, &sh_idx, &sh_val);
}

// Writes the settings of n sequences to their slots' places in the per-slot arrays.
__global__ void sampler_set_kernel(const int32_t *__restrict__ slots, int n,
                                   const unsigned long long *__restrict__ seeds,
                                   const float *__restrict__ temperature,
                                   const int32_t *__restrict__ top_k,
                                   const float *__restrict__ top_p, const float *__restrict__ min_p,
                                   unsigned long long *rng_out, float *temperature_out,
                                   int32_t *top_k_out, float *top_p_out, float *min_p_out)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    int s = slots[i];
    rng_out[s] = seeds[i];
    temperature_out[s] = temperature[i];
    top_k_out[s] = top_k[i];
    top_p_out[s] = top_p[i];
    min_p_out[s] = min_p[i];
}

}  // namespace jb

using namespace jb;

// The most candidates a row can keep without the caller's scratch.
extern "C" int jb_sample_small_cap() { return CHUNK_KEEP; }

// Whether a row with temperature > 0 and this top_k over V logits goes the long way
// (all candidates sorted in the caller's scratch): top_k off or above what a chunk's
// list keeps, or so many chunks that their lists do not fit the merge.  The test is
// the kernel's own (sample_kernel); callers size their scratch by it.
extern "C" int jb_sample_needs_big(int V, int top_k)
{
    int chunks = (V + CHUNK - 1) / CHUNK;
    bool short_way = top_k > 0 && top_k <= CHUNK_KEEP && top_k < V && chunks * CHUNK_KEEP <= MERGE_CAP;
    return short_way ? 0 : 1;
}

// The sampling settings of n sequences (arrays of n values on the device) to the
// places of their slots in the per-slot arrays; each random sequence starts at its
// seed (src/llm/sample.c:118).  An ordinary launch: it runs after all that is ahead
// of it in the stream.
extern "C" int jb_sampler_set(const int32_t *slots, int n, const unsigned long long *seeds,
                              const float *temperature, const int32_t *top_k, const float *top_p,
                              const float *min_p, unsigned long long *rng_out,
                              float *temperature_out, int32_t *top_k_out, float *top_p_out,
                              float *min_p_out, cudaStream_t st)
{
    if (n <= 0)
        return JB_OK;
    sampler_set_kernel<<<(n + 127) / 128, 128, 0, st>>>(slots, n, seeds, temperature, top_k, top_p,
                                                        min_p, rng_out, temperature_out, top_k_out,
                                                        top_p_out, min_p_out);
    return launch_status();
}

// 64-bit words of scratch that jb_sample wants for rows x V logits.
extern "C" long long jb_sample_scratch(int rows, int V)
{
    if (rows <= 0 || V <= 0)
        return 0;
    return (long long)rows * ((V + CHUNK - 1) / CHUNK) * CHUNK_KEEP;
}

// Kernels that jb_sample launches for these arguments (for counting).
extern "C" int jb_sample_launches(int V, long long big_cap, int sampled)
{
    int n = 2;
    if (sampled && big_cap >= V) {
        n += 2;                                         // fill, the blocks' first sort
        for (long long size = 2 * SORT_BLOCK; size <= big_cap; size <<= 1) {
            for (long long stride = size >> 1; stride >= SORT_BLOCK; stride >>= 1)
                n++;
            n++;
        }
    }
    return n;
}

// logits: [rows, V] float.  The per-sequence settings and the random state
// are indexed by row_slot[row] (by the row itself when row_slot is null);
// temperature null means every row takes the first maximum.  chunk_keys:
// jb_sample_scratch(rows, V) words of scratch.  big_keys [rows, big_cap] and
// big_probs [rows, big_cap] are needed only when a row may keep more than
// jb_sample_small_cap() candidates (top_k off or above it); big_cap must then be a
// power of two not below V.  out[row] is the token, or -1 when that scratch was
// needed and not given.
extern "C" int jb_sample(const float *logits, int rows, int V, const int32_t *row_slot,
                         const float *temperature, const int32_t *top_k, const float *top_p,
                         const float *min_p, unsigned long long *rng,
                         unsigned long long *big_keys, float *big_probs, long long big_cap,
                         unsigned long long *chunk_keys, int32_t *out, int32_t *forced,
                         cudaStream_t st)
{
    if (rows <= 0)
        return JB_OK;
    if (V <= 0 || chunk_keys == nullptr || (temperature != nullptr && rng == nullptr))
        return JB_EINVAL;
    if (big_keys != nullptr && (big_probs == nullptr || big_cap < V || (big_cap & (big_cap - 1))))
        return JB_EINVAL;
    int chunks = (V + CHUNK - 1) / CHUNK;
    bool sampled = temperature != nullptr;
    launch(sample_chunks_kernel, (unsigned)(rows * chunks), SAMPLE_THREADS, 0, st, logits, V, chunks,
           (uint64_t *)chunk_keys, sampled ? 0 : 1);
    if (cudaGetLastError() != cudaSuccess)
        return JB_ELAUNCH;
    if (sampled && big_keys != nullptr) {
        long long P = big_cap;
        uint64_t *keys = (uint64_t *)big_keys;
        dim3 per_key((unsigned)((P + SAMPLE_THREADS - 1) / SAMPLE_THREADS), rows);
        dim3 per_block((unsigned)((P + SORT_BLOCK - 1) / SORT_BLOCK), rows);
        dim3 per_pair((unsigned)((P / 2 + SAMPLE_THREADS - 1) / SAMPLE_THREADS), rows);
        launch(sample_fill_kernel, per_key, SAMPLE_THREADS, 0, st, logits, V, row_slot, temperature,
               (const uint64_t *)chunk_keys, chunks, keys, P);
        launch(sort_local_kernel<true>, per_block, SAMPLE_THREADS, 0, st, keys, P, (long long)0);
        for (long long size = 2 * SORT_BLOCK; size <= P; size <<= 1) {
            for (long long stride = size >> 1; stride >= SORT_BLOCK; stride >>= 1)
                launch(sort_global_kernel, per_pair, SAMPLE_THREADS, 0, st, keys, P, size, stride);
            launch(sort_local_kernel<false>, per_block, SAMPLE_THREADS, 0, st, keys, P, size);
        }
        if (cudaGetLastError() != cudaSuccess)
            return JB_ELAUNCH;
    }
    launch(sample_kernel, rows, SAMPLE_THREADS, 0, st, logits, V, row_slot, temperature, top_k, top_p,
           min_p, (uint64_t *)rng, (uint64_t *)big_keys, big_probs, big_cap,
           (const uint64_t *)chunk_keys, chunks, sampled ? CHUNK_KEEP : 1, out, forced);
    return launch_status();
}
