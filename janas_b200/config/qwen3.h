// The Qwen3 dense decoder's typed configuration (see qwen3.cpp).
#pragma once

#include <string>
#include <vector>

#include "registry.h"

namespace jb {

struct Qwen3Config : ArchConfig {
    long long vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0;
    long long num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0;
    long long max_position_embeddings = 0;
    double rms_norm_eps = 0, rope_theta = 0;
    bool tie_word_embeddings = false;
    // layer_types[i] is "full_attention" or "sliding_attention"
    std::vector<std::string> layer_types;
    long long sliding_window = 0;       // 0: no layer slides
    std::vector<int> eos_ids;
    std::string arch = "Qwen3ForCausalLM";

    static Qwen3Config from_json(const Json &config_json);
    void validate() const;

    std::string architecture() const override { return arch; }
    Json to_json() const override;
    ModelSpec to_model_spec() const override;
    std::vector<int> eos_token_ids() const override { return eos_ids; }
};

}  // namespace jb
