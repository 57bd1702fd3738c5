#include "model.h"

#include <set>

namespace jb {

DecoderModel::DecoderModel(const ModelSpec &s, DType dt, Device *d) : spec(s), dtype(dt), dev(d) {
    spec.validate();
    if (dt != F32 && dt != BF16) fail(JB_LLM_EINVAL, "the compute dtype is float32 or bfloat16");
    for (auto &ls : spec.layers)
        blocks.push_back(build_block(ls.block, build_mixer(ls.mixer, dt, d),
                                     build_feed_forward(ls.feed_forward, dt, d),
                                     build_norm(ls.mixer_norm, dt, d), build_norm(ls.ffn_norm, dt, d)));
    final_norm = build_norm(spec.final_norm, dt, d);
    if (final_norm->size() != spec.hidden_size)
        config_error("the final norm's size is not the model's hidden size");
}

void DecoderModel::layer_names(int i, std::string n[4]) const {
    const LayerSpec &ls = spec.layers[(size_t)i];
    n[0] = Part::name(ls.prefix, ls.mixer_name);
    n[1] = Part::name(ls.prefix, ls.ffn_name);
    n[2] = Part::name(ls.prefix, ls.mixer_norm_name);
    n[3] = Part::name(ls.prefix, ls.ffn_norm_name);
}

TensorList DecoderModel::layer_tensors(int i) const {
    std::string n[4];
    layer_names(i, n);
    TensorList t;
    const Block &b = *blocks[(size_t)i];
    b.mixer_norm->tensors(n[2], t);
    b.mixer->tensors(n[0], t);
    b.ffn_norm->tensors(n[3], t);
    b.feed_forward->tensors(n[1], t);
    return t;
}

TensorList DecoderModel::top_tensors() const {
    TensorList t;
    t.emplace_back(spec.embedding_name, TensorSpec{{spec.vocab_size, spec.hidden_size}, EMBEDDING, false});
    final_norm->tensors(spec.final_norm_name, t);
    t.emplace_back(spec.head_name, TensorSpec{{spec.vocab_size, spec.hidden_size}, MATRIX, spec.tie_embeddings});
    return t;
}

TensorList DecoderModel::tensors() const {
    TensorList top = top_tensors();
    TensorList t;
    t.push_back(top.front());
    for (size_t i = 0; i < blocks.size(); i++) {
        TensorList l = layer_tensors((int)i);
        t.insert(t.end(), l.begin(), l.end());
    }
    t.insert(t.end(), top.begin() + 1, top.end());
    std::set<std::string> seen;
    for (auto &kv : t)
        if (!seen.insert(kv.first).second) config_error("two parts of the model name the tensor " + kv.first);
    return t;
}

void DecoderModel::load_top(TensorMap &t) {
    embedding = Part::take(t, spec.embedding_name);
    auto it = t.find(spec.head_name);
    if (it != t.end()) {
        head = it->second;
        t.erase(it);
    } else if (spec.tie_embeddings) {
        head = embedding;
    } else {
        fail(JB_LLM_EOPEN, "tensor " + spec.head_name + " is missing");
    }
    final_norm->load(spec.final_norm_name, t);
}

void DecoderModel::load_layer(int i, TensorMap &t) {
    std::string n[4];
    layer_names(i, n);
    Block &b = *blocks[(size_t)i];
    b.mixer_norm->load(n[2], t);
    b.mixer->load(n[0], t);
    b.ffn_norm->load(n[3], t);
    b.feed_forward->load(n[1], t);
}

void DecoderModel::load_checkpoint(const Checkpoint &ckpt) {
    if (!dev) fail(JB_LLM_EFAIL, "a model without a device cannot load weights");
    check_weights(ckpt, tensors());
    auto bring = [&](const TensorList &list, TensorMap &m) {
        for (auto &kv : list) {
            auto it = ckpt.tensors.find(kv.first);
            if (it == ckpt.tensors.end()) continue;     // optional and absent
            m[kv.first] = upload_tensor(*dev, it->second, resident_dtype(it->second.dtype, kv.second.kind, dtype));
        }
    };
    TensorMap m;
    bring(top_tensors(), m);
    load_top(m);
    for (size_t i = 0; i < blocks.size(); i++) {
        TensorMap lm;
        bring(layer_tensors((int)i), lm);
        load_layer((int)i, lm);
    }
    dev->sync();
    loaded = true;
}

void DecoderModel::load_random(unsigned long long seed) {
    if (!dev) fail(JB_LLM_EFAIL, "a model without a device cannot make weights");
    tensors();      // checks the names
    auto make = [&](const TensorList &list, TensorMap &m) {
        for (auto &kv : list) {
            if (kv.second.optional) continue;
            m[kv.first] = random_tensor(*dev, kv.first, kv.second, seed, dtype);
        }
    };
    TensorMap m;
    make(top_tensors(), m);
    load_top(m);
    for (size_t i = 0; i < blocks.size(); i++) {
        TensorMap lm;
        make(layer_tensors((int)i), lm);
        load_layer((int)i, lm);
    }
    dev->sync();
    loaded = true;
}

size_t DecoderModel::weight_bytes() const {
    size_t total = head.bytes();
    std::set<int> used;
    for (auto &e : spec.run_order) used.insert(e.layer);
    for (int layer : used) {
        const Block &b = *blocks[(size_t)layer];
        total += b.mixer->weight_bytes() + b.feed_forward->weight_bytes() + b.mixer_norm->weight_bytes() +
                 b.ffn_norm->weight_bytes();
    }
    return total + final_norm->weight_bytes();
}

std::vector<KVSpec> DecoderModel::kv_specs() const {
    std::vector<KVSpec> out;
    for (auto &e : spec.run_order)
        out.push_back(e.cache_of >= 0 ? KVSpec() : blocks[(size_t)e.layer]->mixer->kv_spec());
    return out;
}

std::vector<StateSpec> DecoderModel::state_specs() const {
    std::vector<StateSpec> out;
    for (auto &e : spec.run_order) out.push_back(blocks[(size_t)e.layer]->mixer->state_spec());
    return out;
}

void DecoderModel::prepare(long long n_positions) {
    for (auto &b : blocks) b->mixer->prepare(n_positions);
}

bool DecoderModel::supports(StepKind kind) const {
    for (auto &b : blocks)
        if (!b->mixer->supports(kind)) return false;
    return true;
}

bool DecoderModel::graph_safe() const {
    for (auto &b : blocks)
        if (!b->mixer->graph_safe() || !b->feed_forward->graph_safe()) return false;
    return true;
}

Buf DecoderModel::forward(StepContext &ctx, const int32_t *tokens, std::vector<LayerCache> &caches,
                          const int32_t *want_rows, long long n_want) {
    if (!loaded) fail(JB_LLM_EFAIL, "the model has no weights yet");
    Device &d = *ctx.dev;
    long long n = ctx.n_rows;
    Buf x = ops::embed(d, embedding, tokens, n);
    Stack pending;
    for (size_t e = 0; e < spec.run_order.size(); e++) {
        blocks[(size_t)spec.run_order[e].layer]->forward(ctx, x.as<float>(), pending, caches[e]);
        if (ctx.trace) {
            if (pending) {
                ops::add_(d, x.as<float>(), n, spec.hidden_size, pending);
                pending = Stack();
            }
            std::vector<float> host((size_t)n * (size_t)spec.hidden_size);
            cuda_check(cudaMemcpyAsync(host.data(), x.ptr, host.size() * 4, cudaMemcpyDeviceToHost, d.stream),
                       "copying the residual stream");
            d.sync();
            ctx.trace->push_back(std::move(host));
        }
    }
    if (n_want == 0) return Buf();
    bool all = n_want < 0;
    Buf h = final_norm->apply(ctx, x.as<float>(), n, ctx.dtype, pending ? &pending : nullptr,
                              all ? nullptr : want_rows, all ? 0 : n_want);
    Stack lg = ops::linear(d, h.ptr, ctx.dtype, all ? n : n_want, spec.hidden_size, head, true);
    return std::move(lg.buf);
}

}  // namespace jb
