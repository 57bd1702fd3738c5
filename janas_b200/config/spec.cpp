#include "spec.h"

namespace jb {

void config_error(const std::string &m, int code) { throw Error(code, m); }

long long PartSpec::get_int(const std::string &k) const {
    const Json &v = params.get(k);
    if (v.is_null()) config_error(kind + ": parameter " + k + " is missing");
    if (!v.is_number() || !v.whole()) config_error(kind + ": parameter " + k + " must be a whole number");
    return v.as_int();
}

long long PartSpec::get_int(const std::string &k, long long dflt) const {
    return has(k) ? get_int(k) : dflt;
}

double PartSpec::get_double(const std::string &k) const {
    const Json &v = params.get(k);
    if (!v.is_number()) config_error(kind + ": parameter " + k + " must be a number");
    return v.as_double();
}

PartSpec PartSpec::get_part(const std::string &k) const {
    const Json &v = params.get(k);
    if (!v.is_object()) config_error(kind + ": parameter " + k + " must be a part");
    return PartSpec::from_json(v);
}

Json PartSpec::to_json() const {
    Json j = Json::object();
    j.set("kind", kind);
    j.set("params", params);
    return j;
}

PartSpec PartSpec::from_json(const Json &j) {
    if (!j.is_object() || !j.get("kind").is_string())
        config_error("a part is written {\"kind\": name, \"params\": {...}}", JB_LLM_EINVAL);
    PartSpec p;
    p.kind = j.get("kind").as_string();
    if (j.get("params").is_object()) p.params = j.get("params");
    return p;
}

void ModelSpec::validate() const {
    if (hidden_size <= 0 || vocab_size <= 0 || max_positions <= 0)
        config_error("hidden_size, vocab_size and max_positions must be positive");
    if (layers.empty()) config_error("a model needs at least one layer");
    if (run_order.empty()) config_error("the run order is empty");
    for (size_t at = 0; at < run_order.size(); at++) {
        const RunEntry &e = run_order[at];
        if (e.layer < 0 || e.layer >= (int)layers.size())
            config_error(fmt("run order entry %zu names layer %d, the model has %zu", at, e.layer,
                             layers.size()));
        if (e.cache_of >= 0) {
            if (e.cache_of >= (int)at)
                config_error(fmt("run order entry %zu reads the cache of entry %d, which has not run "
                                 "before it", at, e.cache_of));
            if (run_order[e.cache_of].cache_of >= 0)
                config_error(fmt("run order entry %zu reads the cache of entry %d, which owns none",
                                 at, e.cache_of));
        }
    }
}

Json ModelSpec::to_json() const {
    Json j = Json::object();
    j.set("architecture", architecture);
    j.set("hidden_size", hidden_size);
    j.set("vocab_size", vocab_size);
    j.set("max_positions", max_positions);
    Json ls = Json::array();
    for (auto &l : layers) {
        Json o = Json::object();
        o.set("block", l.block);
        o.set("mixer", l.mixer.to_json());
        o.set("feed_forward", l.feed_forward.to_json());
        o.set("mixer_norm", l.mixer_norm.to_json());
        o.set("ffn_norm", l.ffn_norm.to_json());
        o.set("prefix", l.prefix);
        o.set("mixer_name", l.mixer_name);
        o.set("ffn_name", l.ffn_name);
        o.set("mixer_norm_name", l.mixer_norm_name);
        o.set("ffn_norm_name", l.ffn_norm_name);
        ls.push(o);
    }
    j.set("layers", ls);
    Json ro = Json::array();
    for (auto &e : run_order) {
        Json o = Json::object();
        o.set("layer", e.layer);
        o.set("cache_of", e.cache_of >= 0 ? Json(e.cache_of) : Json());
        ro.push(o);
    }
    j.set("run_order", ro);
    j.set("final_norm", final_norm.to_json());
    j.set("tie_embeddings", tie_embeddings);
    j.set("embedding_name", embedding_name);
    j.set("final_norm_name", final_norm_name);
    j.set("head_name", head_name);
    return j;
}

static std::string str_or(const Json &j, const char *k, const std::string &dflt) {
    return j.get(k).is_string() ? j.get(k).as_string() : dflt;
}

ModelSpec ModelSpec::from_json(const Json &j) {
    if (!j.is_object()) config_error("a model spec is a JSON object", JB_LLM_EINVAL);
    ModelSpec s;
    s.architecture = str_or(j, "architecture", "");
    s.hidden_size = j.get("hidden_size").as_int();
    s.vocab_size = j.get("vocab_size").as_int();
    s.max_positions = j.get("max_positions").as_int();
    for (auto &o : j.get("layers").items()) {
        LayerSpec l;
        l.block = str_or(o, "block", "prenorm");
        l.mixer = PartSpec::from_json(o.get("mixer"));
        l.feed_forward = PartSpec::from_json(o.get("feed_forward"));
        l.mixer_norm = PartSpec::from_json(o.get("mixer_norm"));
        l.ffn_norm = PartSpec::from_json(o.get("ffn_norm"));
        l.prefix = str_or(o, "prefix", "");
        l.mixer_name = str_or(o, "mixer_name", l.mixer_name);
        l.ffn_name = str_or(o, "ffn_name", l.ffn_name);
        l.mixer_norm_name = str_or(o, "mixer_norm_name", l.mixer_norm_name);
        l.ffn_norm_name = str_or(o, "ffn_norm_name", l.ffn_norm_name);
        s.layers.push_back(l);
    }
    for (auto &o : j.get("run_order").items()) {
        RunEntry e;
        e.layer = (int)o.get("layer").as_int();
        e.cache_of = o.get("cache_of").is_null() ? -1 : (int)o.get("cache_of").as_int();
        s.run_order.push_back(e);
    }
    s.final_norm = PartSpec::from_json(j.get("final_norm"));
    s.tie_embeddings = j.get("tie_embeddings").as_bool();
    s.embedding_name = str_or(j, "embedding_name", s.embedding_name);
    s.final_norm_name = str_or(j, "final_norm_name", s.final_norm_name);
    s.head_name = str_or(j, "head_name", s.head_name);
    return s;
}

}  // namespace jb
