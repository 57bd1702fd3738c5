// Registries of part kinds: one name -> factory table for each role.
#include <mutex>

#include "part.h"

namespace jb {

const char *step_kind_name(StepKind k) {
    return k == PREFILL ? "prefill" : k == DECODE ? "decode" : "extend";
}

namespace {
struct Tables {
    std::map<std::string, std::map<std::string, PartFactory>> parts;
    std::map<std::string, BlockFactory> blocks;
    std::mutex mu;
};
Tables &raw() {
    static Tables *t = new Tables();
    return *t;
}
Tables &ready() {
    static std::once_flag once;
    std::call_once(once, [] {
        register_builtin_norms();
        register_builtin_positions();
        register_builtin_mixers();
        register_builtin_feed_forwards();
        register_builtin_blocks();
    });
    return raw();
}
bool known_role(const std::string &r) {
    return r == "mixer" || r == "feed_forward" || r == "norm" || r == "position";
}
}  // namespace

void register_part(const std::string &role, const std::string &kind, PartFactory f) {
    if (!known_role(role)) fail(JB_LLM_EINVAL, "no role '" + role + "' (mixer, feed_forward, norm, position)");
    Tables &t = raw();
    std::lock_guard<std::mutex> lock(t.mu);
    t.parts[role][kind] = std::move(f);
}

void register_block(const std::string &kind, BlockFactory f) {
    Tables &t = raw();
    std::lock_guard<std::mutex> lock(t.mu);
    t.blocks[kind] = std::move(f);
}

std::vector<std::string> registered_parts(const std::string &role) {
    Tables &t = ready();
    std::lock_guard<std::mutex> lock(t.mu);
    std::vector<std::string> out;
    if (role == "block") {
        for (auto &kv : t.blocks) out.push_back(kv.first);
    } else {
        for (auto &kv : t.parts[role]) out.push_back(kv.first);
    }
    return out;
}

std::unique_ptr<Part> build_part(const std::string &role, const PartSpec &spec, DType dt, Device *dev) {
    if (!known_role(role)) fail(JB_LLM_EINVAL, "no role '" + role + "' (mixer, feed_forward, norm, position)");
    if (dt != F32 && dt != BF16) fail(JB_LLM_EINVAL, "the compute dtype is float32 or bfloat16");
    PartFactory f;
    {
        Tables &t = ready();
        std::lock_guard<std::mutex> lock(t.mu);
        auto &table = t.parts[role];
        auto it = table.find(spec.kind);
        if (it == table.end()) {
            std::string known;
            for (auto &kv : table) known += (known.empty() ? "" : ", ") + kv.first;
            config_error("no " + role + " of kind '" + spec.kind + "'; registered: " + known);
        }
        f = it->second;
    }
    return f(spec, dt, dev);
}

template <class T>
static std::unique_ptr<T> as_role(std::unique_ptr<Part> p, const char *role, const PartSpec &spec) {
    T *t = dynamic_cast<T *>(p.get());
    if (!t) config_error(std::string("the part registered as ") + role + " '" + spec.kind + "' is not a " + role);
    p.release();
    return std::unique_ptr<T>(t);
}

std::unique_ptr<Mixer> build_mixer(const PartSpec &s, DType dt, Device *d) {
    return as_role<Mixer>(build_part("mixer", s, dt, d), "mixer", s);
}
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec &s, DType dt, Device *d) {
    return as_role<FeedForward>(build_part("feed_forward", s, dt, d), "feed_forward", s);
}
std::unique_ptr<Norm> build_norm(const PartSpec &s, DType dt, Device *d) {
    return as_role<Norm>(build_part("norm", s, dt, d), "norm", s);
}
std::unique_ptr<PositionEncoding> build_position(const PartSpec &s, DType dt, Device *d) {
    return as_role<PositionEncoding>(build_part("position", s, dt, d), "position", s);
}

std::unique_ptr<Block> build_block(const std::string &kind, std::unique_ptr<Mixer> m,
                                   std::unique_ptr<FeedForward> f, std::unique_ptr<Norm> n1,
                                   std::unique_ptr<Norm> n2) {
    BlockFactory bf;
    {
        Tables &t = ready();
        std::lock_guard<std::mutex> lock(t.mu);
        auto it = t.blocks.find(kind);
        if (it == t.blocks.end()) {
            std::string known;
            for (auto &kv : t.blocks) known += (known.empty() ? "" : ", ") + kv.first;
            config_error("no block arrangement '" + kind + "'; registered: " + known);
        }
        bf = it->second;
    }
    return bf(std::move(m), std::move(f), std::move(n1), std::move(n2));
}

DevTensor Part::take(TensorMap &t, const std::string &name) {
    auto it = t.find(name);
    if (it == t.end()) fail(JB_LLM_EOPEN, "tensor " + name + " is missing");
    DevTensor v = it->second;
    t.erase(it);
    return v;
}

DevTensor fuse_rows(Device &dev, std::vector<DevTensor> &mats) {
    if (mats.empty()) fail(JB_LLM_EINVAL, "fuse_rows: nothing to fuse");
    if (mats.size() == 1) return mats[0];
    DType dt = mats[0].dt;
    long long cols = mats[0].shape.at(1), rows = 0;
    for (auto &m : mats) {
        if (m.dt == F32) dt = F32;
        if (m.shape.size() != 2 || m.shape[1] != cols) fail(JB_LLM_EINVAL, "fuse_rows: rows of unequal length");
        rows += m.shape[0];
    }
    dev.make_current();
    DevTensor out = dev.tensor(dt, {rows, cols});
    size_t at = 0;
    for (auto &m : mats) {
        if (jb_convert(m.ptr, m.dt, (char *)out.ptr + at, dt, m.numel(), dev.stream) != 0)
            fail(JB_LLM_EFAIL, "fuse_rows: the copy could not be launched");
        at += (size_t)m.numel() * dtype_size(dt);
    }
    dev.sync();      // the sources are freed when the caller lets go of them
    for (auto &m : mats) m = DevTensor();
    return out;
}

}  // namespace jb
