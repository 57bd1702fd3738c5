// Architecture-neutral description of a decoder: what the engine builds from.
//
// A typed architecture configuration (Qwen3Config) is turned into a ModelSpec.
// The spec is plain data: for every layer it names the mixer, the feed-forward,
// the norms and the block arrangement together with their constants, and
// run_order lists which layers run in which order.  The engine, the cache and
// the weight loader read only this spec, never the architecture's own
// configuration, so that a second architecture adds a configuration class and a
// to_model_spec and nothing else.
//
// The reference keeps the same information in a table row per architecture and
// per-layer fields (struct janas_arch src/llm/arch.h:21-62, struct layer
// src/llm/model_impl.h:36-106); layers that read another layer's keys and values
// are src/llm/model_load.c:1047-1056.
//
// A spec is also JSON (to_json / from_json): that is how a model that is not a
// registered architecture (a test's toy model) reaches the library.
#pragma once

#include <string>
#include <vector>

#include "../core/error.h"
#include "../core/json.h"

namespace jb {

// A configuration that cannot be built: a missing key, a wrong value.  The
// C interface reports it as JB_LLM_EOPEN (an unsupported architecture: EMODEL).
[[noreturn]] void config_error(const std::string &m, int code = JB_LLM_EOPEN);

// One part of a layer: its registered kind and its constants (a JSON object;
// a value may itself be a part, written {"kind": ..., "params": {...}}).
struct PartSpec {
    std::string kind;
    Json params = Json::object();

    bool has(const std::string &k) const { return params.has(k) && !params.get(k).is_null(); }
    long long get_int(const std::string &k) const;            // config_error when absent or not whole
    long long get_int(const std::string &k, long long dflt) const;
    double get_double(const std::string &k) const;
    PartSpec get_part(const std::string &k) const;

    Json to_json() const;
    static PartSpec from_json(const Json &j);
};

// One layer: how its parts are arranged and where its tensors are found.
// prefix is the layer's tensor-name prefix in the checkpoint; the four *_name
// fields are the sub-prefixes of its parts below it.
struct LayerSpec {
    std::string block;
    PartSpec mixer, feed_forward, mixer_norm, ffn_norm;
    std::string prefix;
    std::string mixer_name = "self_attn";
    std::string ffn_name = "mlp";
    std::string mixer_norm_name = "input_layernorm";
    std::string ffn_norm_name = "post_attention_layernorm";
};

// One entry of the run order: run `layer` (its weights).  A layer may be named
// by several entries; every entry is a place of its own in the cache.  With
// cache_of >= 0 (the index of an earlier entry) the entry's mixer writes nothing
// and reads that entry's cache.
struct RunEntry {
    int layer = 0;
    int cache_of = -1;
};

struct ModelSpec {
    std::string architecture;
    long long hidden_size = 0, vocab_size = 0, max_positions = 0;
    std::vector<LayerSpec> layers;
    std::vector<RunEntry> run_order;
    PartSpec final_norm;
    bool tie_embeddings = false;
    std::string embedding_name = "model.embed_tokens.weight";
    std::string final_norm_name = "model.norm";
    std::string head_name = "lm_head.weight";

    void validate() const;          // config_error
    Json to_json() const;
    static ModelSpec from_json(const Json &j);
};

}  // namespace jb
