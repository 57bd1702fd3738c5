// Typed configuration of the Qwen3 dense decoder, read from its config.json.
//
// The keys are the architecture's own (the ones the reference's converter reads
// for a Hugging Face model folder, tools/hf2gguf.c:245-277, and the
// hyper-parameters its loader requires, src/llm/model_load.c:817-836).  No size
// has a default in code except where the reference has one: head_dim falls
// back to hidden_size / num_attention_heads (tools/hf2gguf.c:262-263) and
// tie_word_embeddings to false (tools/hf2gguf.c:264-265).
//
// What Qwen3 dense does not have is refused here instead of being ignored:
// attention biases, RoPE scaling, an activation other than SiLU (the reference's
// table row for qwen3 sets no flag: src/llm/arch.c:11).  A sliding window
// (use_sliding_window, sliding_window, max_window_layers, layer_types) is
// honoured: a sliding layer sees the last sliding_window positions, itself
// included (src/llm/attention.c:736-739).
#include "qwen3.h"

#include <set>

namespace jb {

static const char *kRequired[] = {
    "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
    "num_key_value_heads", "max_position_embeddings", "rms_norm_eps", "rope_theta"};

static const char *FULL = "full_attention";
static const char *SLIDING = "sliding_attention";

static long long as_int(const Json &d, const char *key) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number() || !v.whole())
        config_error(std::string("config.json: ") + key + " must be a whole number, got " + v.dump());
    return v.as_int();
}

static double as_float(const Json &d, const char *key) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number())
        config_error(std::string("config.json: ") + key + " must be a number, got " + v.dump());
    return v.as_double();
}

Qwen3Config Qwen3Config::from_json(const Json &d) {
    std::string missing;
    for (const char *k : kRequired)
        if (d.get(k).is_null()) missing += (missing.empty() ? "" : ", ") + std::string(k);
    if (!missing.empty()) config_error("config.json: missing " + missing);

    Qwen3Config c;
    c.hidden_size = as_int(d, "hidden_size");
    c.num_attention_heads = as_int(d, "num_attention_heads");
    if (c.num_attention_heads <= 0) config_error("config.json: num_attention_heads must be positive");
    if (!d.get("head_dim").is_null()) {
        c.head_dim = as_int(d, "head_dim");
    } else {
        if (c.hidden_size % c.num_attention_heads)
            config_error("config.json: no head_dim, and hidden_size is not a multiple of "
                         "num_attention_heads");
        c.head_dim = c.hidden_size / c.num_attention_heads;
    }
    if (d.get("attention_bias").as_bool())
        config_error("config.json: attention_bias is set; the Qwen3 dense decoder has no attention "
                     "biases");
    const Json &rs = d.get("rope_scaling");
    if (!rs.is_null() && !(rs.is_object() && rs.size() == 0))
        config_error("config.json: rope_scaling is set; only plain RoPE is built");
    if (d.has("hidden_act") && !d.get("hidden_act").is_null() &&
        !(d.get("hidden_act").is_string() && d.get("hidden_act").as_string() == "silu"))
        config_error("config.json: hidden_act " + d.get("hidden_act").dump() + "; Qwen3 uses silu");
    c.num_hidden_layers = as_int(d, "num_hidden_layers");
    if (c.num_hidden_layers <= 0 || c.num_hidden_layers > 100000)
        config_error("config.json: num_hidden_layers must be positive");

    bool use_window = d.get("use_sliding_window").as_bool();
    const Json &lt = d.get("layer_types");
    if (!lt.is_null()) {
        if (!lt.is_array() || (long long)lt.size() != c.num_hidden_layers)
            config_error(fmt("config.json: layer_types has %zu entries for %lld layers", lt.size(),
                             c.num_hidden_layers));
        for (auto &t : lt.items()) {
            if (!t.is_string() || (t.as_string() != FULL && t.as_string() != SLIDING))
                config_error("config.json: unknown layer type " + t.dump());
            c.layer_types.push_back(t.as_string());
        }
    } else if (use_window) {
        long long first = d.get("max_window_layers").is_null() ? 0 : as_int(d, "max_window_layers");
        for (long long i = 0; i < c.num_hidden_layers; i++)
            c.layer_types.push_back(i >= first ? SLIDING : FULL);
    } else {
        c.layer_types.assign((size_t)c.num_hidden_layers, FULL);
    }
    bool any_sliding = false;
    for (auto &t : c.layer_types) any_sliding |= t == SLIDING;
    if (any_sliding) {
        if (d.get("sliding_window").is_null())
            config_error("config.json: sliding layers but no sliding_window");
        c.sliding_window = as_int(d, "sliding_window");
        if (c.sliding_window <= 0) config_error("config.json: sliding_window must be positive");
    }

    const Json &eos = d.get("eos_token_id");
    if (eos.is_array()) {
        for (auto &e : eos.items()) c.eos_ids.push_back((int)e.as_int());
    } else if (eos.is_number()) {
        c.eos_ids.push_back((int)eos.as_int());
    }
    const Json &archs = d.get("architectures");
    if (archs.is_array() && archs.size() > 0 && archs[0].is_string()) c.arch = archs[0].as_string();

    c.vocab_size = as_int(d, "vocab_size");
    c.intermediate_size = as_int(d, "intermediate_size");
    c.num_key_value_heads = as_int(d, "num_key_value_heads");
    c.max_position_embeddings = as_int(d, "max_position_embeddings");
    c.rms_norm_eps = as_float(d, "rms_norm_eps");
    c.rope_theta = as_float(d, "rope_theta");
    c.tie_word_embeddings = d.get("tie_word_embeddings").as_bool();
    c.validate();
    return c;
}

void Qwen3Config::validate() const {
    struct { const char *name; long long v; } sizes[] = {
        {"vocab_size", vocab_size}, {"hidden_size", hidden_size},
        {"intermediate_size", intermediate_size}, {"num_hidden_layers", num_hidden_layers},
        {"num_attention_heads", num_attention_heads}, {"num_key_value_heads", num_key_value_heads},
        {"head_dim", head_dim}, {"max_position_embeddings", max_position_embeddings}};
    for (auto &s : sizes)
        if (s.v <= 0 || s.v > (1ll << 40))
            config_error(std::string("config.json: ") + s.name + " must be positive");
    // src/llm/model_load.c:827 (heads a multiple of KV heads)
    if (num_attention_heads % num_key_value_heads)
        config_error("config.json: num_attention_heads must be a multiple of num_key_value_heads");
    if (head_dim % 2) config_error("config.json: head_dim must be even (RoPE rotates pairs)");
    // what the attention kernels take; said here so that a folder is refused as
    // a configuration before any part is built
    if (head_dim % 16 || head_dim > 512)
        config_error(fmt("config.json: head_dim %lld: this library's attention kernels take head "
                         "sizes from 16 to 512 in steps of 16", head_dim));
    if (!(rms_norm_eps > 0)) config_error("config.json: rms_norm_eps must be positive");
    if (!(rope_theta > 0)) config_error("config.json: rope_theta must be positive");
    if ((long long)layer_types.size() != num_hidden_layers)
        config_error("layer_types must name every layer");
}

Json Qwen3Config::to_json() const {
    Json d = Json::object();
    Json a = Json::array();
    a.push(arch);
    d.set("architectures", a);
    d.set("model_type", "qwen3");
    d.set("vocab_size", vocab_size);
    d.set("hidden_size", hidden_size);
    d.set("intermediate_size", intermediate_size);
    d.set("num_hidden_layers", num_hidden_layers);
    d.set("num_attention_heads", num_attention_heads);
    d.set("num_key_value_heads", num_key_value_heads);
    d.set("head_dim", head_dim);
    d.set("hidden_act", "silu");
    d.set("max_position_embeddings", max_position_embeddings);
    d.set("rms_norm_eps", rms_norm_eps);
    d.set("rope_theta", rope_theta);
    d.set("rope_scaling", Json());
    d.set("attention_bias", false);
    d.set("tie_word_embeddings", tie_word_embeddings);
    bool any_sliding = false;
    for (auto &t : layer_types) any_sliding |= t == SLIDING;
    if (any_sliding) {
        d.set("use_sliding_window", true);
        d.set("sliding_window", sliding_window);
        Json lt = Json::array();
        for (auto &t : layer_types) lt.push(t);
        d.set("layer_types", lt);
    } else {
        d.set("use_sliding_window", false);
        d.set("sliding_window", Json());
    }
    if (eos_ids.size() == 1) d.set("eos_token_id", eos_ids[0]);
    else if (eos_ids.size() > 1) {
        Json e = Json::array();
        for (int t : eos_ids) e.push(t);
        d.set("eos_token_id", e);
    }
    return d;
}

// The decoder as parts: pre-norm blocks of GQA attention (per-head q/k RMSNorm,
// NeoX RoPE over the whole head) and a SwiGLU feed-forward, all RMSNorm with one
// eps (src/llm/model.c:743-796, src/llm/model_attn.c:93-101).
ModelSpec Qwen3Config::to_model_spec() const {
    PartSpec norm{"rmsnorm", Json::object()};
    norm.params.set("size", hidden_size);
    norm.params.set("eps", rms_norm_eps);
    PartSpec rope{"rope_neox", Json::object()};
    rope.params.set("rotary_dim", head_dim);
    rope.params.set("theta", rope_theta);
    rope.params.set("max_positions", max_position_embeddings);
    PartSpec ffn{"swiglu", Json::object()};
    ffn.params.set("hidden_size", hidden_size);
    ffn.params.set("intermediate_size", intermediate_size);

    ModelSpec s;
    s.architecture = arch;
    s.hidden_size = hidden_size;
    s.vocab_size = vocab_size;
    s.max_positions = max_position_embeddings;
    for (long long i = 0; i < num_hidden_layers; i++) {
        PartSpec mixer{"gqa_attention", Json::object()};
        mixer.params.set("hidden_size", hidden_size);
        mixer.params.set("num_heads", num_attention_heads);
        mixer.params.set("num_kv_heads", num_key_value_heads);
        mixer.params.set("head_dim", head_dim);
        mixer.params.set("qk_norm_eps", rms_norm_eps);
        mixer.params.set("window", layer_types[(size_t)i] == SLIDING ? sliding_window : 0);
        mixer.params.set("position", rope.to_json());
        LayerSpec l;
        l.block = "prenorm";
        l.mixer = mixer;
        l.feed_forward = ffn;
        l.mixer_norm = norm;
        l.ffn_norm = norm;
        l.prefix = fmt("model.layers.%lld", i);
        s.layers.push_back(l);
        s.run_order.push_back(RunEntry{(int)i, -1});
    }
    s.final_norm = norm;
    s.tie_embeddings = tie_word_embeddings;
    s.validate();
    return s;
}

void register_qwen3() {
    register_architecture("Qwen3ForCausalLM", "qwen3", [](const Json &d) {
        return std::unique_ptr<ArchConfig>(new Qwen3Config(Qwen3Config::from_json(d)));
    });
}

}  // namespace jb
