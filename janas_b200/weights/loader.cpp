#include "loader.h"

#include <algorithm>
#include <cstring>
#include <set>

namespace jb {

const char *kind_name(TensorKind k) {
    switch (k) {
        case MATRIX: return "matrix";
        case EMBEDDING: return "embedding";
        case NORM: return "norm";
        case INT_TABLE: return "int_table";
    }
    return "?";
}

TensorKind parse_kind(const std::string &s) {
    if (s == "matrix") return MATRIX;
    if (s == "embedding") return EMBEDDING;
    if (s == "norm") return NORM;
    if (s == "int_table") return INT_TABLE;
    fail(JB_LLM_EINVAL, "unknown tensor kind '" + s + "'");
}

static Json shape_json(const std::vector<long long> &s) {
    Json a = Json::array();
    for (auto v : s) a.push(v);
    return a;
}

Json tensor_list_json(const TensorList &l) {
    Json a = Json::array();
    for (auto &kv : l) {
        Json o = Json::object();
        o.set("name", kv.first);
        o.set("shape", shape_json(kv.second.shape));
        o.set("kind", kind_name(kv.second.kind));
        o.set("optional", kv.second.optional);
        a.push(o);
    }
    return a;
}

TensorList tensor_list_from_json(const Json &j) {
    TensorList l;
    if (!j.is_array()) fail(JB_LLM_EINVAL, "a tensor list is a JSON array");
    for (auto &o : j.items()) {
        TensorSpec s;
        for (auto &v : o.get("shape").items()) s.shape.push_back(v.as_int());
        s.kind = o.get("kind").is_string() ? parse_kind(o.get("kind").as_string()) : MATRIX;
        s.optional = o.get("optional").as_bool();
        l.emplace_back(o.get("name").as_string(), s);
    }
    return l;
}

Json WeightMismatch::to_json() const {
    Json o = Json::object();
    Json m = Json::array(), u = Json::array(), ws = Json::array(), wt = Json::array();
    for (auto &n : missing) m.push(n);
    for (auto &n : unexpected) u.push(n);
    for (auto &s : wrong_shape) {
        Json e = Json::object();
        e.set("name", s.name);
        e.set("want", shape_json(s.want));
        e.set("got", shape_json(s.got));
        ws.push(e);
    }
    for (auto &t : wrong_type) {
        Json e = Json::object();
        e.set("name", t.first);
        e.set("stored", t.second);
        wt.push(e);
    }
    o.set("missing", m);
    o.set("unexpected", u);
    o.set("wrong_shape", ws);
    o.set("wrong_type", wt);
    return o;
}

DType resident_dtype(const std::string &stored, TensorKind kind, DType compute) {
    if (kind == INT_TABLE) return I32;
    if (compute == F32 || stored == "F32") return F32;
    return BF16;
}

static std::string shape_text(const std::vector<long long> &s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); i++) t += (i ? ", " : "") + std::to_string(s[i]);
    return t + "]";
}

void check_weights(const Checkpoint &ckpt, const TensorList &expected) {
    std::vector<std::string> missing, unexpected;
    std::vector<WeightMismatch::Shape> wrong_shape;
    std::vector<std::pair<std::string, std::string>> wrong_type;
    std::set<std::string> names;
    for (auto &kv : expected) {
        names.insert(kv.first);
        auto it = ckpt.tensors.find(kv.first);
        if (it == ckpt.tensors.end()) {
            if (!kv.second.optional) missing.push_back(kv.first);
            continue;
        }
        const TensorInfo &info = it->second;
        if (info.shape != kv.second.shape)
            wrong_shape.push_back({kv.first, kv.second.shape, info.shape});
        bool is_int = info.dtype == "I32" || info.dtype == "I64";
        if ((kv.second.kind == INT_TABLE) != is_int) wrong_type.emplace_back(kv.first, info.dtype);
    }
    for (auto &n : ckpt.names)
        if (!names.count(n)) unexpected.push_back(n);
    if (missing.empty() && unexpected.empty() && wrong_shape.empty() && wrong_type.empty()) return;
    std::sort(missing.begin(), missing.end());
    std::sort(unexpected.begin(), unexpected.end());
    std::string msg = ckpt.model_dir + ": the weights do not match the configuration";
    auto join = [](const std::vector<std::string> &v) {
        std::string t;
        for (size_t i = 0; i < v.size(); i++) t += (i ? ", " : "") + v[i];
        return t;
    };
    if (!missing.empty()) msg += fmt("\n  missing (%zu): ", missing.size()) + join(missing);
    if (!unexpected.empty()) msg += fmt("\n  unexpected (%zu): ", unexpected.size()) + join(unexpected);
    for (auto &s : wrong_shape)
        msg += "\n  wrong shape: " + s.name + " is " + shape_text(s.got) + ", expected " + shape_text(s.want);
    for (auto &t : wrong_type) msg += "\n  wrong type: " + t.first + " is stored as " + t.second;
    WeightMismatch e(msg);
    e.missing = missing;
    e.unexpected = unexpected;
    e.wrong_shape = wrong_shape;
    e.wrong_type = wrong_type;
    throw e;
}

// ------------------------------------------------------------- conversions
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {       // round to nearest even
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1);
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// Converts `count` elements starting at element `first`.
static void convert_range(const TensorInfo &info, DType resident, long long first, long long count,
                          void *dst) {
    const uint8_t *src = info.data + (size_t)first * (size_t)stored_size(info.dtype);
    const std::string &st = info.dtype;
    if ((st == "F32" && resident == F32) || (st == "BF16" && resident == BF16) ||
        (st == "I32" && resident == I32)) {
        memcpy(dst, src, (size_t)count * dtype_size(resident));
    } else if (st == "BF16" && resident == F32) {
        const uint16_t *s = (const uint16_t *)src;
        float *d = (float *)dst;
        for (long long i = 0; i < count; i++) d[i] = bf16_to_f32(s[i]);
    } else if (st == "F16" && resident == F32) {
        const uint16_t *s = (const uint16_t *)src;
        float *d = (float *)dst;
        for (long long i = 0; i < count; i++) d[i] = f16_to_f32(s[i]);
    } else if (st == "F16" && resident == BF16) {
        const uint16_t *s = (const uint16_t *)src;
        uint16_t *d = (uint16_t *)dst;
        for (long long i = 0; i < count; i++) d[i] = f32_to_bf16(f16_to_f32(s[i]));
    } else if (st == "I64" && resident == I32) {
        const int64_t *s = (const int64_t *)src;
        int32_t *d = (int32_t *)dst;
        for (long long i = 0; i < count; i++) {
            if (s[i] > INT32_MAX || s[i] < INT32_MIN)
                fail(JB_LLM_EOPEN, info.path + ": " + info.name + " does not fit int32");
            d[i] = (int32_t)s[i];
        }
    } else {
        fail(JB_LLM_EOPEN, info.path + ": " + info.name + " stored as " + st + " cannot be kept as " +
                               dtype_name(resident));
    }
}

void convert_tensor(const TensorInfo &info, DType resident, void *dst) {
    convert_range(info, resident, 0, info.count(), dst);
}

DevTensor upload_tensor(Device &dev, const TensorInfo &info, DType resident) {
    dev.make_current();
    DevTensor t = dev.tensor(resident, info.shape);
    long long n = info.count();
    size_t esz = dtype_size(resident);
    bool same = (info.dtype == "F32" && resident == F32) || (info.dtype == "BF16" && resident == BF16) ||
                (info.dtype == "I32" && resident == I32);
    if (same) {
        if (n) cuda_check(cudaMemcpy(t.ptr, info.data, (size_t)n * esz, cudaMemcpyHostToDevice),
                          "copying a tensor to the device");
        return t;
    }
    const long long chunk = 4 << 20;     // elements
    std::vector<uint8_t> stage((size_t)std::min(n, chunk) * esz);
    for (long long a = 0; a < n; a += chunk) {
        long long c = std::min(chunk, n - a);
        convert_range(info, resident, a, c, stage.data());
        cuda_check(cudaMemcpy((uint8_t *)t.ptr + (size_t)a * esz, stage.data(), (size_t)c * esz,
                              cudaMemcpyHostToDevice), "copying a tensor to the device");
    }
    return t;
}

// FNV-1a over the name, mixed with the seed: the tensor's own random stream
static unsigned long long tensor_seed(unsigned long long seed, const std::string &name) {
    unsigned long long h = 1469598103934665603ull ^ (seed * 0x9E3779B97F4A7C15ull);
    for (unsigned char c : name) { h ^= c; h *= 1099511628211ull; }
    return h;
}

DevTensor random_tensor(Device &dev, const std::string &name, const TensorSpec &spec,
                        unsigned long long seed, DType dt) {
    if (spec.kind == INT_TABLE) fail(JB_LLM_EINVAL, name + ": no random rule for integer tables");
    if (dt != F32 && dt != BF16) fail(JB_LLM_EINVAL, "random weights are made as bfloat16 or float32");
    dev.make_current();
    DevTensor t = dev.tensor(dt, spec.shape);
    float mean = spec.kind == NORM ? 1.0f : 0.0f, std = spec.kind == NORM ? 0.1f : 0.02f;
    int rc = jb_fill_normal(t.ptr, (int)dt, t.numel(), tensor_seed(seed, name), mean, std, dev.stream);
    if (rc != 0) fail(JB_LLM_EFAIL, name + ": the random fill could not be launched");
    return t;
}

}  // namespace jb
