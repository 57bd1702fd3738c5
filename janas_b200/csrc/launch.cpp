#include "launch.h"

#include <algorithm>
#include <atomic>
#include <vector>

#include "../cache/cache.h"
#include "kernels.h"

namespace jb {
namespace ops {

static std::atomic<long long> g_launches{0};

long long launches() { return g_launches.load(); }
void count_launches(long long n) { g_launches += n; }

static void check(int code, const char *what, int kernels = 1) {
    if (code == 0) {
        g_launches += kernels;
        return;
    }
    if (code == -1) fail(JB_LLM_EINVAL, std::string(what) + ": the kernel does not take these sizes or types");
    cudaError_t e = cudaGetLastError();
    fail(JB_LLM_EFAIL, fmt("%s: the launch failed (code %d%s%s)", what, code, e != cudaSuccess ? ": " : "",
                           e != cudaSuccess ? cudaGetErrorString(e) : ""));
}

static void need_float(DType dt, const char *what) {
    if (dt != F32 && dt != BF16) fail(JB_LLM_EINVAL, std::string(what) + ": float32 or bfloat16 is needed");
}

static int as_int(long long v, const char *what) {
    if (v < 0 || v > 0x7fffffffll) fail(JB_LLM_EINVAL, std::string(what) + ": too large for the kernels");
    return (int)v;
}

int attention_chunk() { return jb_attention_chunk(); }
int sample_small_cap() { return jb_sample_small_cap(); }
bool sample_needs_big(int vocab, int top_k) { return jb_sample_needs_big(vocab, top_k) != 0; }

// ------------------------------------------------------------------ row-wise
Buf embed(Device &d, const DevTensor &table, const int32_t *tokens, long long n) {
    need_float(table.dt, "embedding table");
    long long dm = table.shape.at(1);
    Buf x = d.pool.get((size_t)n * (size_t)dm * 4);
    check(jb_embed(table.ptr, table.dt, tokens, x.as<float>(), as_int(n, "rows"), as_int(dm, "width"),
                   d.stream), "embed");
    return x;
}

Buf rmsnorm(Device &d, float *x, long long n, long long dm, const DevTensor &w, float eps, DType out_dt,
            const Stack *delta, const int32_t *rows, long long n_out) {
    need_float(w.dt, "norm weight");
    need_float(out_dt, "norm output");
    if (w.numel() != dm) fail(JB_LLM_EINVAL, "rmsnorm: the weight's length is not the rows' width");
    if (delta && rows) {
        add_(d, x, n, dm, *delta);
        delta = nullptr;
    }
    if (delta && (delta->n != n || delta->m != dm))
        fail(JB_LLM_EINVAL, "rmsnorm: delta's shape is not x's");
    long long outs = rows ? n_out : n;
    Buf out = d.pool.get((size_t)outs * (size_t)dm * dtype_size(out_dt));
    check(jb_rmsnorm(x, delta ? delta->data() : nullptr, delta ? delta->S : 0,
                     delta ? delta->stride() : 0, rows, w.ptr, w.dt, out.ptr, out_dt, as_int(outs, "rows"),
                     as_int(dm, "width"), eps, d.stream), "rmsnorm");
    return out;
}

void add_(Device &d, float *x, long long n, long long dm, const Stack &delta) {
    if (delta.n != n || delta.m != dm) fail(JB_LLM_EINVAL, "add: delta's shape is not x's");
    check(jb_rmsnorm(x, delta.data(), delta.S, delta.stride(), nullptr, nullptr, 0, nullptr, 0,
                     as_int(n, "rows"), as_int(dm, "width"), 0.0f, d.stream), "add");
}

Buf swiglu(Device &d, const Stack &gu, DType out_dt) {
    if (gu.m % 2) fail(JB_LLM_EINVAL, "swiglu: the gate_up width must be even");
    long long ff = gu.m / 2;
    Buf out = d.pool.get((size_t)gu.n * (size_t)ff * dtype_size(out_dt));
    check(jb_swiglu(gu.data(), gu.S, gu.stride(), out.ptr, out_dt, as_int(gu.n, "rows"), as_int(ff, "width"),
                    d.stream), "swiglu");
    return out;
}

void rope_table(Device &d, const float *inv, int half, long long n_pos, float *cs, float *sn) {
    check(jb_rope_table(cs, sn, inv, as_int(n_pos, "positions"), half, d.stream), "rope_table");
}

// ------------------------------------------------------------------ products
int linear_parts(long long n, long long m, long long k) {
    return jb_gemm_tc_splits((int)n, (int)m, (int)k);
}

Stack linear(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &w,
             bool whole, bool force_simt, int splits) {
    need_float(a_dt, "activations");
    need_float(w.dt, "weight");
    if (w.shape.size() != 2 || w.shape[1] != k)
        fail(JB_LLM_EINVAL, "linear: the weight's rows are not as long as the activations'");
    long long m = w.shape[0];
    Stack out;
    out.n = n;
    out.m = m;
    int ni = as_int(n, "rows"), mi = as_int(m, "features"), ki = as_int(k, "width");
    if (!force_simt && n > 0 && a_dt == BF16 && w.dt == BF16 && jb_gemm_tc_ok(a, w.ptr, ni, mi, ki)) {
        out.S = whole ? 1 : (splits > 0 ? splits : jb_gemm_tc_splits(ni, mi, ki));
        out.buf = d.pool.get((size_t)out.S * (size_t)n * (size_t)m * 4);
        check(jb_gemm_tc(a, w.ptr, out.data(), ni, mi, ki, out.S, d.stream), "linear (tcgen05)");
        return out;
    }
    out.S = 1;
    out.buf = d.pool.get((size_t)n * (size_t)m * 4);
    long long need = jb_gemm_simt_scratch(ni, mi, ki);
    Buf scratch;
    if (need > 0) scratch = d.pool.get((size_t)need * 4);
    check(jb_gemm_simt(a, a_dt, w.ptr, w.dt, out.data(), ni, mi, ki, scratch.as<float>(), d.stream),
          "linear", need > 0 ? 2 : 1);
    return out;
}

Buf linear_swiglu(Device &d, const void *a, DType a_dt, long long n, long long k, const DevTensor &gu) {
    if (gu.shape.size() != 2 || gu.shape[1] != k)
        fail(JB_LLM_EINVAL, "linear_swiglu: the weight's rows are not as long as the activations'");
    if (gu.shape[0] % 2 || n == 0 || a_dt != BF16 || gu.dt != BF16 ||
        !jb_gemm_tc_ok(a, gu.ptr, (int)n, (int)gu.shape[0], (int)k))
        return Buf();
    long long ff = gu.shape[0] / 2;
    Buf out = d.pool.get((size_t)n * (size_t)ff * 2);
    check(jb_gemm_tc_swiglu(a, gu.ptr, out.ptr, as_int(n, "rows"), as_int(ff, "features"), as_int(k, "width"),
                            d.stream), "linear_swiglu (tcgen05)");
    return out;
}

// ----------------------------------------------------------------- attention
Buf qk_norm_rope_append(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w, float eps,
                        const float *cs, const float *sn, const int32_t *row_pos, const int32_t *row_seq,
                        const AttnCache &c, const AttnGeometry &g, DType out_dt) {
    long long width = (long long)(g.nh + 2 * g.nkv) * g.hd;
    if (qkv.m != width) fail(JB_LLM_EINVAL, "qk_norm_rope_append: qkv is not heads + 2 kv_heads wide");
    int w_dt = 0;
    if (q_w) {
        if (!k_w || q_w->dt != k_w->dt || q_w->numel() != g.hd || k_w->numel() != g.hd)
            fail(JB_LLM_EINVAL, "qk_norm_rope_append: q and k norm weights of one type and the head's size");
        need_float(q_w->dt, "q_norm weight");
        w_dt = q_w->dt;
    }
    bool append = c.writes && c.k != nullptr;
    if (append && c.dt != out_dt) fail(JB_LLM_EINVAL, "qk_norm_rope_append: the cache is of another type");
    Buf q = d.pool.get((size_t)qkv.n * (size_t)g.nh * (size_t)g.hd * dtype_size(out_dt));
    check(jb_qk_norm_rope_append(qkv.data(), qkv.S, qkv.stride(), q_w ? q_w->ptr : nullptr,
                                 k_w ? k_w->ptr : nullptr, w_dt, eps, cs, sn, cs ? g.hd / 2 : 0, row_pos,
                                 row_seq, c.block_table, c.bt_stride, q.ptr, append ? c.k : nullptr,
                                 append ? c.v : nullptr, out_dt, as_int(qkv.n, "rows"), g.nh, g.nkv, g.hd,
                                 d.stream), "qk_norm_rope_append");
    return q;
}

int attention_block_positions(int nh, int nkv) { return jb_attn_tc_block_positions(nh, nkv); }
bool attention_tc_ok(int nh, int nkv, int hd) { return jb_attn_tc_ok(nh, nkv, hd) != 0; }

Buf attention_blocks(Device &d, const long long *row0, const long long *pos0, const long long *len,
                     int n_seqs, int per, int *n_blocks) {
    struct B { int32_t row, count, pos, seq; };
    std::vector<B> rows;
    for (int i = 0; i < n_seqs; i++)
        for (long long a = 0; a < len[i]; a += per)
            rows.push_back({(int32_t)(row0[i] + a), (int32_t)std::min<long long>(per, len[i] - a),
                            (int32_t)(pos0[i] + a), (int32_t)i});
    // the runs that end latest see the most keys and take longest: they start first
    std::stable_sort(rows.begin(), rows.end(),
                     [](const B &x, const B &y) { return x.pos + x.count > y.pos + y.count; });
    *n_blocks = (int)rows.size();
    Buf out = d.pool.get(std::max<size_t>(rows.size() * sizeof(B), 16));
    d.upload(out.ptr, rows.data(), rows.size() * sizeof(B));
    return out;
}

// Into how many CTAs the chunks of one (token, KV head) pair are cut.  A CTA costs
// about three chunks' time to set up, and CTAs beyond the device's places (two per
// SM) come in waves: the cut that finishes first by that estimate.
static int decode_parts(long long pairs, int chunks, int places) {
    int best = 1;
    double best_t = -1;
    for (int parts = 1; parts <= chunks; parts++) {
        int per_cta = (chunks + parts - 1) / parts;
        long long ctas = pairs * ((chunks + per_cta - 1) / per_cta);
        long long waves = (ctas + places - 1) / places;
        double t = (double)waves * (3.0 + per_cta);
        if (best_t < 0 || t < best_t) { best = parts; best_t = t; }
    }
    return best;
}

static const size_t ATT_SCRATCH_BYTES = (size_t)256 << 20;

Buf attention(Device &d, const void *q, long long n, const AttnCache &c, const AttnGeometry &g,
              const int32_t *row_pos, const int32_t *row_seq, int max_chunks, const int32_t *blocks,
              int n_blocks, bool decode, bool force_simt) {
    need_float(c.dt, "attention");
    int ni = as_int(n, "rows");
    Buf out = d.pool.get((size_t)n * (size_t)g.nh * (size_t)g.hd * dtype_size(c.dt));
    bool tc = !force_simt && c.dt == BF16 && (decode || blocks != nullptr) && attention_tc_ok(g.nh, g.nkv, g.hd);
    if (tc && !decode) {
        check(jb_attn_tc_prefill(q, c.k, c.v, c.n_pages, blocks, n_blocks, c.block_table, c.bt_stride,
                                 out.ptr, ni, g.nh, g.nkv, g.hd, g.window, g.scale, d.stream),
              "attention (tcgen05, prefill)");
        return out;
    }
    int parts = max_chunks, per_cta = 1;
    if (tc) {
        // CTAs per (token, KV head): each runs over per_cta chunks and leaves one partial
        if (jb_attn_tc_decode_runs(g.nh, g.nkv, g.hd))
            parts = decode_parts(std::min<long long>(n, 4096) * g.nkv, max_chunks, 2 * d.sm_count);
        per_cta = (max_chunks + parts - 1) / parts;
        parts = (max_chunks + per_cta - 1) / per_cta;
    }
    long long per_row = jb_attention_scratch(1, g.nh, g.hd, parts);
    long long rows_per_call = std::max<long long>(1, std::min<long long>(n, (long long)(ATT_SCRATCH_BYTES / 4) /
                                                                                 std::max<long long>(per_row, 1)));
    Buf scratch = d.pool.get((size_t)per_row * (size_t)rows_per_call * 4);
    for (long long row0 = 0; row0 < n; row0 += rows_per_call) {
        int cnt = (int)std::min<long long>(rows_per_call, n - row0);
        if (tc) {
            check(jb_attn_tc_decode(q, c.k, c.v, c.n_pages, row_pos, row_seq, c.block_table, c.bt_stride,
                                    scratch.as<float>(), ni, (int)row0, cnt, g.nh, g.nkv, g.hd, g.window,
                                    g.scale, max_chunks, per_cta, d.stream), "attention (tcgen05, decode)");
            check(jb_attention_merge(scratch.as<float>(), row_pos, out.ptr, c.dt, (int)row0, cnt, g.nh, g.hd,
                                     g.window, parts, per_cta, d.stream), "attention merge");
        } else {
            check(jb_attention(q, c.k, c.v, c.dt, row_pos, row_seq, c.block_table, c.bt_stride,
                               scratch.as<float>(), out.ptr, (int)row0, cnt, g.nh, g.nkv, g.hd, g.window,
                               g.scale, max_chunks, d.stream), "attention", 2);
        }
    }
    return out;
}

Buf attention_decode_qkv(Device &d, const Stack &qkv, const DevTensor *q_w, const DevTensor *k_w, float eps,
                         const float *cs, const float *sn, const AttnCache &c, const AttnGeometry &g,
                         const int32_t *row_pos, const int32_t *row_seq, int max_chunks) {
    if (c.dt != BF16 || !c.k || !jb_attn_tc_decode_runs(g.nh, g.nkv, g.hd)) return Buf();
    long long width = (long long)(g.nh + 2 * g.nkv) * g.hd;
    if (qkv.m != width) fail(JB_LLM_EINVAL, "attention: qkv is not heads + 2 kv_heads wide");
    int w_dt = 0;
    if (q_w) {
        if (!k_w || q_w->dt != k_w->dt) fail(JB_LLM_EINVAL, "attention: q and k norm weights of one type");
        w_dt = q_w->dt;
    }
    long long n = qkv.n;
    int ni = as_int(n, "rows");
    int parts = decode_parts(std::min<long long>(n, 4096) * g.nkv, max_chunks, 2 * d.sm_count);
    int per_cta = (max_chunks + parts - 1) / parts;
    parts = (max_chunks + per_cta - 1) / per_cta;
    long long per_row = jb_attention_scratch(1, g.nh, g.hd, parts);
    long long rows_per_call = std::max<long long>(1, std::min<long long>(n, (long long)(ATT_SCRATCH_BYTES / 4) /
                                                                                 std::max<long long>(per_row, 1)));
    Buf scratch = d.pool.get((size_t)per_row * (size_t)rows_per_call * 4);
    Buf out = d.pool.get((size_t)n * (size_t)g.nh * (size_t)g.hd * 2);
    for (long long row0 = 0; row0 < n; row0 += rows_per_call) {
        int cnt = (int)std::min<long long>(rows_per_call, n - row0);
        int code = jb_attn_tc_decode_qkv(qkv.data(), qkv.S, qkv.stride(), q_w ? q_w->ptr : nullptr,
                                         k_w ? k_w->ptr : nullptr, w_dt, eps, cs, sn, c.k, c.v,
                                         c.writes ? 1 : 0, c.n_pages, row_pos, row_seq, c.block_table,
                                         c.bt_stride, scratch.as<float>(), ni, (int)row0, cnt, g.nh, g.nkv,
                                         g.hd, g.window, g.scale, max_chunks, per_cta, d.stream);
        if (code == -1 && row0 == 0) return Buf();      // an address the kernel's 16-byte loads cannot take
        check(code, "attention (tcgen05, decode, from the product's sums)");
        check(jb_attention_merge(scratch.as<float>(), row_pos, out.ptr, BF16, (int)row0, cnt, g.nh, g.hd,
                                 g.window, parts, per_cta, d.stream), "attention merge");
    }
    return out;
}

// ------------------------------------------------------------------ sampling
void sample(Device &d, const float *logits, int rows, int vocab, const SamplerArrays &s, int32_t *out) {
    if (s.temperature && !s.rng) fail(JB_LLM_EINVAL, "sample: temperature needs the random states");
    Buf chunk_keys = d.pool.get((size_t)std::max<long long>(jb_sample_scratch(rows, vocab), 1) * 8);
    int launches = jb_sample_launches(vocab, s.big_keys ? s.big_cap : 0, s.temperature != nullptr);
    check(jb_sample(logits, rows, vocab, s.row_slot, s.temperature, s.top_k, s.top_p, s.min_p, s.rng,
                    s.big_keys, s.big_probs, s.big_keys ? s.big_cap : 0,
                    (unsigned long long *)chunk_keys.ptr, out, s.forced, d.stream), "sample", launches);
}

int gemm_tc_error() { return jb_gemm_tc_error(); }
int attn_tc_error() { return jb_attn_tc_error(); }

}  // namespace ops
}  // namespace jb
