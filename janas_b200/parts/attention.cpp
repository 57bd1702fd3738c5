// Grouped-query attention with optional per-head q/k RMSNorm, a position
// encoding and an optional sliding window.
//
// In order: q, k, v products without biases; per head, RMSNorm of q and of k with
// one weight vector for all heads, before the rotation; the rotation; K and V into
// the cache at the row's position; causal attention, head h reading KV head
// h / (heads / kv_heads), scores scaled by 1/sqrt(head size); the output product
// (src/llm/model_attn.c:75-146,224-285; src/llm/attention.c:874-875,1012).  With a
// window w a token at position p sees positions p + 1 - w .. p
// (src/llm/attention.c:736-739).
#include <cmath>

#include "part.h"

namespace jb {

namespace {

// params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (null: no
// q/k norm), window (0: none), position (a part)
class GQAAttention : public Mixer {
public:
    GQAAttention(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        g_.nh = (int)s.get_int("num_heads");
        g_.nkv = (int)s.get_int("num_kv_heads");
        g_.hd = (int)s.get_int("head_dim");
        qk_norm_ = s.has("qk_norm_eps");
        qk_eps_ = qk_norm_ ? (float)s.get_double("qk_norm_eps") : 0.0f;
        g_.window = (int)s.get_int("window", 0);
        if (hidden_ <= 0 || g_.nh <= 0 || g_.nkv <= 0) config_error("gqa_attention: sizes must be positive");
        if (g_.nh % g_.nkv) config_error("gqa_attention: num_heads must be a multiple of num_kv_heads");
        if (g_.hd % 16 || g_.hd < 16 || g_.hd > 512)
            config_error(fmt("gqa_attention: head_dim %d: the kernels take head sizes from 16 to 512 in "
                             "steps of 16", g_.hd));
        if (g_.window < 0) config_error("gqa_attention: window must not be negative");
        position_ = build_position(s.get_part("position"), dt, d);
        if (position_->rotary_dim() != 0 && position_->rotary_dim() != g_.hd)
            config_error(fmt("gqa_attention: only the whole head can be rotated (rotary_dim %d, "
                             "head_dim %d)", position_->rotary_dim(), g_.hd));
        g_.scale = (float)(1.0 / std::sqrt((double)g_.hd));
    }

    // ------------------------------------------------------------- weights
    void tensors(const std::string &p, TensorList &out) const override {
        long long hd = g_.hd;
        out.emplace_back(name(p, "q_proj.weight"), TensorSpec{{g_.nh * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "k_proj.weight"), TensorSpec{{g_.nkv * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "v_proj.weight"), TensorSpec{{g_.nkv * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "o_proj.weight"), TensorSpec{{hidden_, g_.nh * hd}, MATRIX, false});
        if (qk_norm_) {
            out.emplace_back(name(p, "q_norm.weight"), TensorSpec{{hd}, NORM, false});
            out.emplace_back(name(p, "k_norm.weight"), TensorSpec{{hd}, NORM, false});
        }
        position_->tensors(name(p, "position"), out);
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> qkv = {take(t, name(p, "q_proj.weight")), take(t, name(p, "k_proj.weight")),
                                      take(t, name(p, "v_proj.weight"))};
        w_qkv_ = fuse_rows(*dev, qkv);
        w_o_ = take(t, name(p, "o_proj.weight"));
        if (qk_norm_) {
            q_norm_ = take(t, name(p, "q_norm.weight"));
            k_norm_ = take(t, name(p, "k_norm.weight"));
            if (q_norm_.dt != k_norm_.dt) {
                // one kernel reads both: the wider type for both
                std::vector<DevTensor *> both = {&q_norm_, &k_norm_};
                for (DevTensor *w : both) {
                    if (w->dt == F32) continue;
                    DevTensor wide = dev->tensor(F32, w->shape);
                    if (jb_convert(w->ptr, w->dt, wide.ptr, F32, w->numel(), dev->stream) != 0)
                        fail(JB_LLM_EFAIL, "gqa_attention: widening a norm weight failed");
                    dev->sync();
                    *w = wide;
                }
            }
        }
        position_->load(name(p, "position"), t);
    }

    size_t weight_bytes() const override {
        return w_qkv_.bytes() + w_o_.bytes() + q_norm_.bytes() * (qk_norm_ ? 2 : 0);
    }

    // --------------------------------------------------------------- cache
    KVSpec kv_spec() const override { return KVSpec{g_.nkv, g_.hd, g_.window}; }

    void prepare(long long n_positions) override {
        position_->prepare(n_positions);
        chunk_ = ops::attention_chunk();
    }

    // Every kind of step, with a window too: the pages a window group gives back
    // after a step are those that the sequence's NEXT token cannot see, and tokens
    // appended later see no further back than that one.
    bool supports(StepKind) const override { return true; }

    // everything that changes from step to step is read from device arrays, so a
    // captured decode step can be replayed
    bool graph_safe() const override { return true; }

    // ------------------------------------------------------------- forward
    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (ctx.max_pos >= position_->n_positions())
            fail(JB_LLM_EINVAL, fmt("position %lld is beyond the %lld positions the encoding was prepared "
                                    "for", ctx.max_pos, position_->n_positions()));
        if (!chunk_) chunk_ = ops::attention_chunk();
        long long n = ctx.n_rows;
        const DevTensor *qw = qk_norm_ ? &q_norm_ : nullptr, *kw = qk_norm_ ? &k_norm_ : nullptr;
        Stack qkv = ops::linear(d, h, ctx.dtype, n, hidden_, w_qkv_);
        int max_chunks = (int)(ctx.max_pos / chunk_ + 1);
        if (g_.window) max_chunks = std::min(max_chunks, (g_.window - 1) / chunk_ + 2);
        Buf a;
        if (ctx.kind == DECODE && ctx.dtype == BF16) {
            // one new token per sequence: the attention kernel makes q and the new key
            // and value from the product's sums itself, where it takes the sizes
            a = ops::attention_decode_qkv(d, qkv, qw, kw, qk_eps_, position_->cos(), position_->sin(),
                                          cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks);
        }
        if (!a) {
            Buf q = ops::qk_norm_rope_append(d, qkv, qw, kw, qk_eps_, position_->cos(), position_->sin(),
                                             ctx.row_pos, ctx.row_seq, cache.kv, g_, ctx.dtype);
            qkv.buf.reset();
            bool decode = ctx.kind == DECODE;
            const int32_t *blocks = nullptr;
            int n_blocks = 0;
            if (!decode && ctx.dtype == BF16 && ops::attention_tc_ok(g_.nh, g_.nkv, g_.hd) &&
                !ctx.seq_len.empty()) {
                // runs of consecutive positions, for the tensor-core kernel; the same
                // for every layer of the step with this grouping of heads
                int per = ops::attention_block_positions(g_.nh, g_.nkv);
                std::string key = "attention_blocks/" + std::to_string(per);
                auto it = ctx.extras.find(key);
                if (it == ctx.extras.end()) {
                    StepContext::Extra e;
                    e.buf = ops::attention_blocks(d, ctx.seq_row0.data(), ctx.seq_pos0.data(),
                                                  ctx.seq_len.data(), ctx.n_seqs, per, &e.n);
                    it = ctx.extras.emplace(key, std::move(e)).first;
                }
                blocks = it->second.buf.as<int32_t>();
                n_blocks = it->second.n;
            }
            a = ops::attention(d, q.ptr, n, cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks, blocks,
                               n_blocks, decode);
        }
        return ops::linear(d, a.ptr, ctx.dtype, n, (long long)g_.nh * g_.hd, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("position", position_->info());
        o.set("position_kind", position_->spec.kind);
        return o;
    }

private:
    long long hidden_;
    ops::AttnGeometry g_;
    bool qk_norm_;
    float qk_eps_;
    std::unique_ptr<PositionEncoding> position_;
    DevTensor w_qkv_, w_o_, q_norm_, k_norm_;
    int chunk_ = 0;
};

}  // namespace

void register_builtin_mixers() {
    register_part("mixer", "gqa_attention", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new GQAAttention(s, dt, d));
    });
}

}  // namespace jb
