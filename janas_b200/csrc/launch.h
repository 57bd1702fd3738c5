// The kernels as checked C++ calls over device memory.
//
// Each function takes what the kernel takes, gets its output and scratch from
// the device's pool of temporaries, launches on the device's stream and throws a
// jb::Error when the kernel library refuses the sizes (JB_LLM_EINVAL) or the
// launch fails (JB_LLM_EFAIL).  There is no CPU fallback and no library model
// code behind these functions.
//
// Conventions: the residual stream and every matrix product's output are
// float32.  A product's output is a stack [S, n, m] of S partial sums whose sum
// over S is the result (S = 1 unless the product was split over k); the kernels
// that consume a product add the partial sums in the order 0 .. S-1.
#pragma once

#include <cstdint>

#include "../engine/device.h"

namespace jb {

// float32 partial sums [S, n, m]
struct Stack {
    Buf buf;
    int S = 0;
    long long n = 0, m = 0;
    float *data() const { return (float *)buf.ptr; }
    long long stride() const { return n * m; }
    explicit operator bool() const { return S > 0; }
};

namespace ops {

// how many of the library's kernels have been launched (for measurements)
long long launches();
void count_launches(long long n);

int attention_chunk();
int sample_small_cap();
bool sample_needs_big(int vocab, int top_k);

// x[j, :] = table[tokens[j], :] as float32 [n, dm]
Buf embed(Device &d, const DevTensor &table, const int32_t *tokens, long long n);

// RMSNorm of the rows of x (float32 [n, dm]).  With delta, x is first updated in
// place, x += delta[0] + ... + delta[S-1].  With rows (n_out int32 indices on the
// device) only those rows are normalized and returned, in that order; delta and
// rows together: the add runs first, as a launch of its own.
Buf rmsnorm(Device &d, float *x, long long n, long long dm, const DevTensor &weight, float eps,
            DType out_dt, const Stack *delta, const int32_t *rows, long long n_out);
void add_(Device &d, float *x, long long n, long long dm, const Stack &delta);

// SiLU(gate) * up for a stack [S, n, 2 ff] whose columns are [gate | up]
Buf swiglu(Device &d, const Stack &gate_up, DType out_dt);

// cos and sin of (float)p * inv_freq[i] for p < n_pos: two float32 [n_pos, half]
void rope_table(Device &d, const float *inv_freq_dev, int half, long long n_pos, float *cos_out,
                float *sin_out);

// a [n, k] . weight[m, k]^T as a stack of float32 partial sums.  bfloat16 operands
// whose rows are a multiple of 8 long go to the tensor-core kernel (which may cut
// k into S parts); everything else goes to the plain multiply-add kernel, S = 1.
// whole: S = 1 in every case.
Stack linear(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &weight,
             bool whole = false, bool force_simt = false, int splits = 0);
// Into how many parts of k the tensor-core product is cut when the caller leaves it open.
int linear_parts(long long n, long long m, long long k);
// SiLU(a . gate^T) * (a . up^T) in one tensor-core kernel; an empty Buf when the
// kernel does not take the operands.  Output bfloat16 [n, ff].
Buf linear_swiglu(Device &d, const void *a, DType a_dt, long long n, long long k,
                  const DevTensor &gate_up);

struct AttnGeometry {
    int nh = 0, nkv = 0, hd = 0, window = 0;
    float scale = 1.0f;
};

// what the attention kernels see of the cache and of the step's index arrays
struct AttnCache {
    void *k = nullptr, *v = nullptr;       // [pages, kv_heads, PAGE, head_dim]
    long long n_pages = 0;
    DType dt = F32;
    const int32_t *block_table = nullptr;  // [sequences, bt_stride]
    int bt_stride = 0;
    bool writes = true;
};

// Per-head RMSNorm of q and k (when weights are given), NeoX rotation by the rows'
// positions (when tables are given), K and V appended to the cache pages (when the
// cache writes).  qkv: stack [S, n, (heads + 2 kv_heads) head_dim].  Returns q
// [n, heads, head_dim] in out_dt.
Buf qk_norm_rope_append(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w,
                        float eps, const float *cos, const float *sin, const int32_t *row_pos,
                        const int32_t *row_seq, const AttnCache &c, const AttnGeometry &g,
                        DType out_dt);

// The blocks a prefill step is cut into for the tensor-core kernel: int32
// [blocks, 4] = first row, positions, the first row's position, sequence;
// uploaded to a temporary.  n_blocks comes back.
Buf attention_blocks(Device &d, const long long *seq_row0, const long long *seq_pos0,
                     const long long *seq_len, int n_seqs, int positions_per_block, int *n_blocks);
int attention_block_positions(int nh, int nkv);
bool attention_tc_ok(int nh, int nkv, int hd);

// Causal GQA attention of every row over its sequence's cache pages: q [n, heads,
// hd] of the cache's dtype -> out of the same shape and dtype.  max_chunks: the
// most chunks of attention_chunk() positions that any row's range touches.
// bfloat16 heads of 64 or 128 values run on the tensor cores when the caller says
// how the rows are arranged: decode (every row is the one new token of its
// sequence) or blocks (from attention_blocks).
Buf attention(Device &d, const void *q, long long n, const AttnCache &c, const AttnGeometry &g,
              const int32_t *row_pos, const int32_t *row_seq, int max_chunks, const int32_t *blocks,
              int n_blocks, bool decode, bool force_simt = false);

// qk_norm_rope_append and attention(decode) in one kernel, from the q,k,v product's
// partial sums; an empty Buf where the kernel does not take these sizes and types.
Buf attention_decode_qkv(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w,
                         float eps, const float *cos, const float *sin, const AttnCache &c,
                         const AttnGeometry &g, const int32_t *row_pos, const int32_t *row_seq,
                         int max_chunks);

struct SamplerArrays {
    const int32_t *row_slot = nullptr;
    const float *temperature = nullptr;   // null: every row takes its first maximum
    const int32_t *top_k = nullptr;
    const float *top_p = nullptr, *min_p = nullptr;
    unsigned long long *rng = nullptr;
    unsigned long long *big_keys = nullptr;   // [rows, big_cap] or null
    float *big_probs = nullptr;
    long long big_cap = 0;
    int32_t *forced = nullptr;
};
// One token per row of logits [rows, V] into out (int32 [rows] on the device).
void sample(Device &d, const float *logits, int rows, int vocab, const SamplerArrays &s, int32_t *out);

// 0, or which bounded wait of a tensor-core kernel ran out since the last call
// (the kernels' output is then not valid).  Both synchronize the device.
int gemm_tc_error();
int attn_tc_error();

}  // namespace ops
}  // namespace jb
