#include "registry.h"

#include <algorithm>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <sys/stat.h>

namespace jb {

namespace {
struct Tables {
    std::map<std::string, ArchFactory> by_name;
    std::map<std::string, std::string> by_model_type;
};
// The tables themselves.  Registration writes here directly; readers go through
// ready(), which first puts the built-in architectures in (their registration
// calls register_architecture, so it must not pass through ready() again).
Tables &raw_tables() {
    static Tables *t = new Tables();
    return *t;
}
}  // namespace

void register_architecture(const std::string &name, const std::string &model_type,
                           ArchFactory factory) {
    Tables &t = raw_tables();
    t.by_name[name] = std::move(factory);
    if (!model_type.empty()) t.by_model_type[model_type] = name;
}

static Tables &ready() {
    static std::once_flag once;
    std::call_once(once, [] { register_qwen3(); });
    return raw_tables();
}

std::vector<std::string> known_architectures() {
    std::vector<std::string> out;
    for (auto &kv : ready().by_name) out.push_back(kv.first);
    return out;
}

std::string architecture_name(const Json &d) {
    const Json &archs = d.get("architectures");
    if (archs.is_array() && archs.size() > 0 && archs[0].is_string()) return archs[0].as_string();
    const Json &mt = d.get("model_type");
    if (mt.is_string()) {
        auto &m = ready().by_model_type;
        auto it = m.find(mt.as_string());
        if (it != m.end()) return it->second;
    }
    config_error("config.json names no architecture (architectures, model_type)");
}

std::unique_ptr<ArchConfig> config_from_json(const Json &d) {
    if (!d.is_object()) config_error("config.json: not a JSON object");
    std::string name = architecture_name(d);
    auto &m = ready().by_name;
    auto it = m.find(name);
    if (it == m.end()) {
        std::string known;
        for (auto &kv : m) known += (known.empty() ? "" : ", ") + kv.first;
        config_error("architecture '" + name + "' is not supported; known: " + known, JB_LLM_EMODEL);
    }
    return it->second(d);
}

std::unique_ptr<ArchConfig> config_from_dir(const std::string &model_dir) {
    std::string path = model_dir + "/config.json";
    struct stat st;
    if (stat(path.c_str(), &st) != 0 || !S_ISREG(st.st_mode))
        config_error(model_dir + ": no config.json");
    std::ifstream f(path, std::ios::binary);
    if (!f) config_error(path + ": cannot be read");
    std::stringstream ss;
    ss << f.rdbuf();
    Json d;
    try {
        d = Json::parse(ss.str());
    } catch (const JsonError &e) {
        config_error(path + ": not JSON (" + e.what() + ")");
    }
    if (!d.is_object()) config_error(path + ": not a JSON object");
    return config_from_json(d);
}

}  // namespace jb
