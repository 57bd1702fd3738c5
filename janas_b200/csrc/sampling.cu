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
// Two kernels.  The first cuts every row into chunks of CHUNK logits and lets a
// block sort each chunk (value falling, id rising) and keep its CHUNK_KEEP best;
// with ids in the keys that is exact.  The second has one block per row: it sorts
// the chunks' candidates, which hold the row's CHUNK_KEEP best, and draws.  A row
// that wants more candidates than that (top_k off or above CHUNK_KEEP) goes the
// long way in the second kernel, over all its logits: up to SMALL_CAP candidates
// in shared memory, more in the caller's scratch.
#include "common.cuh"
#include "kernels.h"

namespace jb {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SMALL_CAP = 2048;
constexpr int CHUNK = 4096;          // logits a block of the first kernel sorts
constexpr int CHUNK_KEEP = 64;       // candidates it keeps
constexpr int MERGE_CAP = 4096;      // candidates of all chunks of a row that the second kernel sorts

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

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float *__restrict__ logits, int V, const int32_t *__restrict__ row_slot,
              const float *__restrict__ temperature, const int32_t *__restrict__ top_k,
              const float *__restrict__ top_p, const float *__restrict__ min_p,
              uint64_t *__restrict__ rng, uint64_t *__restrict__ big_keys,
              float *__restrict__ big_probs, long long big_cap,
              const uint64_t *__restrict__ chunk_keys, int chunks, int chunk_kept,
              int32_t *__restrict__ out, int32_t *__restrict__ forced)
{
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    __shared__ uint32_t hist[256];
    __shared__ uint64_t small_keys[MERGE_CAP];
    __shared__ float small_probs[SMALL_CAP];
    __shared__ unsigned n_fill, n_elig, sh_prefix, sh_remain;
    __shared__ unsigned tie_ids[256];

    pdl_trigger();
    pdl_wait();
    int row = blockIdx.x, tid = threadIdx.x;
    int lane = tid & 31, warp = tid >> 5;
    const float *lg = logits + (size_t)row * V;
    int slot = row_slot ? row_slot[row] : row;

    // ---- the short way: the chunks' candidates hold all this row can want
    if (chunk_keys != nullptr) {
        float T = temperature ? temperature[slot] : 0.0f;
        int tk = top_k ? top_k[slot] : 0;
        const uint64_t *src = chunk_keys + (size_t)row * chunks * CHUNK_KEEP;
        if (!(T > 0.0f)) {
            // the first maximum: the least key among the chunks' best
            uint64_t best = ~0ull;
            for (int c = tid; c < chunks; c += SAMPLE_THREADS)
                best = min(best, src[(size_t)c * CHUNK_KEEP]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
                best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
            if (lane == 0)
                small_keys[warp] = best;
            __syncthreads();
            if (warp == 0) {
                best = small_keys[lane];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
                    best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
                if (lane == 0) {
                    out[row] = (int32_t)(uint32_t)best;
                    if (forced)
                        forced[row] = 0;
                }
            }
            return;
        }
        if (tk > 0 && tk <= chunk_kept && chunk_kept == CHUNK_KEEP && tk < V) {
            // the chunks' lists (each sorted, up to 64 of them) are merged two by two,
            // keeping the best 64 of 128 each time, in place: the warp that merges
            // lists a and a + step writes into a
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
    }

    // ---- the first maximum
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        float v = lg[i];
        if (bi == 0x7fffffff || v > bv) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (lane == 0) {
        red_v[warp] = bv;
        red_i[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
        bv = red_v[lane];
        bi = red_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            red_v[0] = bv;
            red_i[0] = bi;
        }
    }
    __syncthreads();
    float mx = red_v[0];
    int amax = red_i[0];
    float T = temperature ? temperature[slot] : 0.0f;
    if (!(T > 0.0f)) {
        if (tid == 0) {
            out[row] = amax;
            if (forced)
                forced[row] = 0;
        }
        return;
    }

    // ---- the candidates
    float floor_v = mx - 30.0f * T;
    int tk = top_k ? top_k[slot] : 0;
    unsigned K = tk > 0 && tk < V ? (unsigned)tk : (unsigned)V;
    if (tid == 0) {
        n_fill = 0;
        n_elig = 0;
    }
    __syncthreads();
    unsigned mine = 0;
    for (int i = tid; i < V; i += SAMPLE_THREADS)
        mine += lg[i] >= floor_v;
    mine = (unsigned)__reduce_add_sync(0xffffffffu, mine);
    if (lane == 0)
        atomicAdd(&n_elig, mine);
    __syncthreads();
    unsigned E = n_elig;
    unsigned n_sel = E < K ? E : K;
    uint32_t thr = 0;     // with E > K: the key of the K-th largest candidate
    unsigned need_eq = 0;  // and how many candidates equal to it are taken
    if (E > K) {
        uint32_t prefix = 0, mask = 0;
        unsigned remain = K;
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256)
                hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                float v = lg[i];
                uint32_t u = ordered_key(v);
                if (v >= floor_v && (u & mask) == prefix)
                    atomicAdd(&hist[(u >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned above = 0;
                int b = 255;
                for (; b > 0; b--) {
                    if (above + hist[b] >= remain)
                        break;
                    above += hist[b];
                }
                sh_prefix = prefix | ((uint32_t)b << shift);
                sh_remain = remain - above;
            }
            __syncthreads();
            prefix = sh_prefix;
            remain = sh_remain;
            mask |= 255u << shift;
            __syncthreads();
        }
        thr = prefix;
        need_eq = remain;
    }

    bool small = n_sel <= SMALL_CAP;
    uint64_t *keys = small ? small_keys : big_keys + (size_t)row * big_cap;
    float *probs = small ? small_probs : big_probs + (size_t)row * big_cap;
    int P = 1;
    while ((unsigned)P < n_sel)
        P <<= 1;
    if (!small && (big_keys == nullptr || (long long)P > big_cap)) {
        if (tid == 0)
            out[row] = -1;  // no scratch for this many candidates
        return;
    }
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        float v = lg[i];
        if (!(v >= floor_v))
            continue;
        uint32_t u = ordered_key(v);
        if (E > K && u <= thr)
            continue;
        unsigned at = atomicAdd(&n_fill, 1u);
        keys[at] = ((uint64_t)(~u) << 32) | (uint32_t)i;
    }
    __syncthreads();
    if (E > K) {
        // the candidates equal to the K-th: the lowest ids first.  Ranges of
        // SAMPLE_THREADS consecutive ids are looked at together; a range's tied ids
        // are counted in order (ballots), so the ones taken are the lowest.
        unsigned at = n_fill, got = 0;
        __syncthreads();
        for (int base = 0; base < V && got < need_eq; base += SAMPLE_THREADS) {
            int i = base + tid;
            bool tie = i < V && lg[i] >= floor_v && ordered_key(lg[i]) == thr;
            unsigned ballot = __ballot_sync(0xffffffffu, tie);
            if (lane == 0)
                tie_ids[warp] = __popc(ballot);
            __syncthreads();
            unsigned before = 0, total = 0;
            for (int w = 0; w < SAMPLE_THREADS / 32; w++) {
                unsigned c = tie_ids[w];
                before += w < warp ? c : 0;
                total += c;
            }
            unsigned rank = got + before + __popc(ballot & ((1u << lane) - 1));
            if (tie && rank < need_eq)
                keys[at + rank] = ((uint64_t)(~thr) << 32) | (uint32_t)i;
            got += total;
            __syncthreads();
        }
    }
    for (int i = n_sel + tid; i < P; i += SAMPLE_THREADS)
        keys[i] = ~0ull;
    __syncthreads();
    bitonic_sort(keys, P);

    float top = key_value(~(uint32_t)(keys[0] >> 32));
    for (unsigned i = tid; i < n_sel; i += SAMPLE_THREADS) {
        float l = key_value(~(uint32_t)(keys[i] >> 32));
        probs[i] = expf((l - top) / T);
    }
    __syncthreads();
    if (tid == 0)
        draw(keys, probs, n_sel, top_p ? top_p[slot] : 0.0f, min_p ? min_p[slot] : 0.0f,
             rng + slot, out + row, forced ? forced + row : nullptr);
}

}  // namespace jb


using namespace jb;

extern "C" int jb_sample_small_cap() { return SMALL_CAP; }

// 64-bit words of scratch that jb_sample wants for rows x V logits (0: none, the
// vocabulary is too large for the short way and every row goes the long one).
extern "C" long long jb_sample_scratch(int rows, int V)
{
    long long chunks = (V + CHUNK - 1) / CHUNK;
    if (rows <= 0 || V <= 0 || chunks * CHUNK_KEEP > MERGE_CAP)
        return 0;
    return (long long)rows * chunks * CHUNK_KEEP;
}

// logits: [rows, V] float.  The per-sequence settings and the random state
// are indexed by row_slot[row] (by the row itself when row_slot is null);
// temperature null means every row takes the first maximum.  chunk_keys:
// jb_sample_scratch(rows, V) words of scratch (or null: every row goes the long
// way).  big_keys [rows, big_cap] and big_probs [rows, big_cap] are needed only
// when a row may keep more than jb_sample_small_cap() candidates; big_cap must
// then be a power of two not below V.  out[row] is the token, or -1 when that
// scratch was needed and not given.
extern "C" int jb_sample(const float *logits, int rows, int V, const int32_t *row_slot,
                         const float *temperature, const int32_t *top_k, const float *top_p,
                         const float *min_p, unsigned long long *rng,
                         unsigned long long *big_keys, float *big_probs, long long big_cap,
                         unsigned long long *chunk_keys, int32_t *out, int32_t *forced,
                         cudaStream_t st)
{
    if (rows <= 0)
        return JB_OK;
    if (V <= 0 || (temperature != nullptr && rng == nullptr))
        return JB_EINVAL;
    int chunks = (V + CHUNK - 1) / CHUNK;
    if (chunk_keys != nullptr && jb_sample_scratch(rows, V) == 0)
        chunk_keys = nullptr;
    int kept = temperature == nullptr ? 1 : CHUNK_KEEP;      // greedy: a chunk's best is enough
    if (chunk_keys != nullptr) {
        launch(sample_chunks_kernel, (unsigned)(rows * chunks), SAMPLE_THREADS, 0, st, logits, V,
               chunks, (uint64_t *)chunk_keys, temperature == nullptr ? 1 : 0);
        if (cudaGetLastError() != cudaSuccess)
            return JB_ELAUNCH;
    }
    launch(sample_kernel, rows, SAMPLE_THREADS, 0, st, logits, V, row_slot, temperature, top_k, top_p,
           min_p, (uint64_t *)rng, (uint64_t *)big_keys, big_probs, big_cap,
           (const uint64_t *)chunk_keys, chunks, kept, out, forced);
    return launch_status();
}
