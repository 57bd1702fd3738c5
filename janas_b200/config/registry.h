// One registry from an architecture's name to its configuration class.
//
// config.json names the architecture (architectures[0], else model_type); the
// class found here reads the file's keys and turns them into a ModelSpec from
// which the one generic decoder is built.  The reference looks the name up in a
// static table in the same way and fails with "architecture ... not supported"
// (src/llm/arch.c:10-66, src/llm/model_load.c:800-804).
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "spec.h"

namespace jb {

// What a configuration class must offer to be registered.
struct ArchConfig {
    virtual ~ArchConfig() = default;
    virtual std::string architecture() const = 0;
    // the architecture's own config.json keys, every one written out
    virtual Json to_json() const = 0;
    virtual ModelSpec to_model_spec() const = 0;
    virtual std::vector<int> eos_token_ids() const { return {}; }
};

using ArchFactory = std::function<std::unique_ptr<ArchConfig>(const Json &config_json)>;

// Makes `name` (as config.json spells it) known; model_type ("" for none) is
// the fallback key for folders that give no architectures list.
void register_architecture(const std::string &name, const std::string &model_type,
                           ArchFactory factory);
std::vector<std::string> known_architectures();
std::string architecture_name(const Json &config_json);
std::unique_ptr<ArchConfig> config_from_json(const Json &config_json);
std::unique_ptr<ArchConfig> config_from_dir(const std::string &model_dir);

// defined in qwen3.cpp; called once by the registry
void register_qwen3();

}  // namespace jb
