// Parts that live outside the library: a mixer, feed-forward, norm or position
// encoding is registered with a callback (jb_register_part in the C interface),
// and the library asks the callback what it would ask a part of its own.  This is
// how a program (or a test) adds a part without changing a file of the library.
//
// The callback gets a method name and its arguments as JSON text and returns JSON
// text (valid until its next call), or null for a failure; an object with an
// "error" member is a failure with a message.  Device memory is passed as
// addresses (whole numbers); the callback's work must be queued on the stream
// whose handle the step's context gives ("stream").
//
//   create      {role, kind, params, dtype}                 -> {id}
//   destroy     {id}
//   tensors     {id, prefix}                                -> {tensors: [{name, shape, kind, optional}]}
//   load        {id, prefix, tensors: {name: {ptr, dtype, shape}}}
//   kv_spec     {id}                                        -> {num_kv_heads, head_dim, window} | {}
//   state_spec  {id}                                        -> {shape, dtype} | {}
//   supports    {id, kind}                                  -> {ok}
//   graph_safe  {id}                                        -> {ok}
//   prepare     {id, n_positions}                           -> (position) {cos, sin, rotary_dim, n_positions}
//   forward     {id, ctx, h, out, [cache]}                  mixer / feed-forward: out is float32 [n, hidden]
//   apply       {id, ctx, x, n, out, out_dtype, delta, rows}    norm
#include "foreign.h"

namespace jb {

namespace {

Json call(const ForeignPartHost &host, const std::string &method, const Json &args) {
    const char *r = host.fn(host.user, method.c_str(), args.dump().c_str());
    if (!r) fail(JB_LLM_EFAIL, "a registered part failed in '" + method + "'");
    Json j = Json::parse(r);
    if (j.is_object() && j.has("error"))
        fail(JB_LLM_EFAIL, "a registered part failed in '" + method + "': " + j.get("error").as_string());
    return j;
}

unsigned long long addr(const void *p) { return (unsigned long long)(uintptr_t)p; }

Json shape_json(const std::vector<long long> &s) {
    Json a = Json::array();
    for (auto v : s) a.push(v);
    return a;
}

Json ctx_json(const StepContext &c) {
    Json o = Json::object();
    o.set("kind", step_kind_name(c.kind));
    o.set("dtype", dtype_name(c.dtype));
    o.set("n_rows", c.n_rows);
    o.set("n_seqs", c.n_seqs);
    o.set("hidden", c.hidden);
    o.set("row_pos", addr(c.row_pos));
    o.set("row_seq", addr(c.row_seq));
    o.set("seq_slot", addr(c.seq_slot));
    Json sl = Json::array(), p0 = Json::array(), ln = Json::array(), r0 = Json::array();
    for (int s : c.seq_slots) sl.push(s);
    for (auto v : c.seq_pos0) p0.push(v);
    for (auto v : c.seq_len) ln.push(v);
    for (auto v : c.seq_row0) r0.push(v);
    o.set("seq_slots", sl);
    o.set("seq_pos0", p0);
    o.set("seq_len", ln);
    o.set("seq_row0", r0);
    o.set("max_pos", c.max_pos);
    o.set("captured", c.captured);
    o.set("stream", addr(c.dev ? c.dev->stream : nullptr));
    o.set("device", c.dev ? c.dev->index : 0);
    return o;
}

Json cache_json(const LayerCache &c) {
    Json o = Json::object();
    o.set("k", addr(c.kv.k));
    o.set("v", addr(c.kv.v));
    o.set("n_pages", c.kv.n_pages);
    o.set("kv_heads", c.kv_heads);
    o.set("head_dim", c.head_dim);
    o.set("page", PAGE);
    o.set("dtype", dtype_name(c.kv.dt));
    o.set("block_table", addr(c.kv.block_table));
    o.set("bt_stride", c.kv.bt_stride);
    o.set("writes", c.kv.writes);
    o.set("state", addr(c.state));
    o.set("state_shape", shape_json(c.state_spec.shape));
    o.set("state_dtype", dtype_name(c.state_spec.dtype));
    o.set("n_slots", c.n_slots);
    return o;
}

// What every foreign part shares: its id over there, its tensors kept alive here.
struct Remote {
    ForeignPartHost host;
    long long id = -1;
    std::vector<DevTensor> held;

    Remote(const ForeignPartHost &h, const std::string &role, const PartSpec &s, DType dt) : host(h) {
        Json a = Json::object();
        a.set("role", role);
        a.set("kind", s.kind);
        a.set("params", s.params);
        a.set("dtype", dtype_name(dt));
        id = call(host, "create", a).get("id").as_int();
    }
    ~Remote() {
        try {
            Json a = Json::object();
            a.set("id", id);
            host.fn(host.user, "destroy", a.dump().c_str());
        } catch (...) {}
    }
    Json ask(const std::string &method, Json a = Json::object()) const {
        a.set("id", id);
        return call(host, method, a);
    }
    void tensors(const std::string &prefix, TensorList &out) const {
        Json a = Json::object();
        a.set("prefix", prefix);
        Json r = ask("tensors", a);
        TensorList l = tensor_list_from_json(r.get("tensors").is_array() ? r.get("tensors") : Json::array());
        out.insert(out.end(), l.begin(), l.end());
    }
    void load(const std::string &prefix, TensorMap &t) {
        TensorList mine;
        tensors(prefix, mine);
        Json ts = Json::object();
        for (auto &kv : mine) {
            auto it = t.find(kv.first);
            if (it == t.end()) {
                if (kv.second.optional) continue;
                fail(JB_LLM_EOPEN, "tensor " + kv.first + " is missing");
            }
            Json e = Json::object();
            e.set("ptr", addr(it->second.ptr));
            e.set("dtype", dtype_name(it->second.dt));
            e.set("shape", shape_json(it->second.shape));
            ts.set(kv.first, e);
            held.push_back(it->second);
            t.erase(it);
        }
        Json a = Json::object();
        a.set("prefix", prefix);
        a.set("tensors", ts);
        ask("load", a);
    }
    size_t bytes() const {
        size_t b = 0;
        for (auto &t : held) b += t.bytes();
        return b;
    }
};

class ForeignMixer : public Mixer {
public:
    ForeignMixer(const ForeignPartHost &h, const PartSpec &s, DType dt, Device *d)
        : Mixer(s, dt, d), r_(h, "mixer", s, dt) {}
    void tensors(const std::string &p, TensorList &out) const override { r_.tensors(p, out); }
    void load(const std::string &p, TensorMap &t) override { r_.load(p, t); }
    size_t weight_bytes() const override { return r_.bytes(); }
    KVSpec kv_spec() const override {
        Json j = r_.ask("kv_spec");
        if (!j.has("num_kv_heads")) return KVSpec();
        return KVSpec{(int)j.get("num_kv_heads").as_int(), (int)j.get("head_dim").as_int(),
                      (int)j.get("window").as_int()};
    }
    StateSpec state_spec() const override {
        Json j = r_.ask("state_spec");
        StateSpec s;
        if (!j.has("shape")) return s;
        for (auto &v : j.get("shape").items()) s.shape.push_back(v.as_int());
        std::string dt = j.get("dtype").is_string() ? j.get("dtype").as_string() : "float32";
        s.dtype = dt == "bfloat16" ? BF16 : dt == "int32" ? I32 : dt == "int64" ? I64 : F32;
        return s;
    }
    void prepare(long long n) override {
        Json a = Json::object();
        a.set("n_positions", n);
        r_.ask("prepare", a);
    }
    bool supports(StepKind k) const override {
        Json a = Json::object();
        a.set("kind", step_kind_name(k));
        return r_.ask("supports", a).get("ok").as_bool();
    }
    bool graph_safe() const override { return r_.ask("graph_safe").get("ok").as_bool(); }
    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Stack out;
        out.S = 1;
        out.n = ctx.n_rows;
        out.m = ctx.hidden;
        out.buf = ctx.dev->pool.get((size_t)out.n * (size_t)out.m * 4);
        Json a = Json::object();
        a.set("ctx", ctx_json(ctx));
        a.set("h", addr(h));
        a.set("out", addr(out.buf.ptr));
        a.set("cache", cache_json(cache));
        r_.ask("forward", a);
        return out;
    }

private:
    Remote r_;
};

class ForeignFeedForward : public FeedForward {
public:
    ForeignFeedForward(const ForeignPartHost &h, const PartSpec &s, DType dt, Device *d)
        : FeedForward(s, dt, d), r_(h, "feed_forward", s, dt) {}
    void tensors(const std::string &p, TensorList &out) const override { r_.tensors(p, out); }
    void load(const std::string &p, TensorMap &t) override { r_.load(p, t); }
    size_t weight_bytes() const override { return r_.bytes(); }
    bool graph_safe() const override { return r_.ask("graph_safe").get("ok").as_bool(); }
    Stack forward(StepContext &ctx, const void *h) override {
        Stack out;
        out.S = 1;
        out.n = ctx.n_rows;
        out.m = ctx.hidden;
        out.buf = ctx.dev->pool.get((size_t)out.n * (size_t)out.m * 4);
        Json a = Json::object();
        a.set("ctx", ctx_json(ctx));
        a.set("h", addr(h));
        a.set("out", addr(out.buf.ptr));
        r_.ask("forward", a);
        return out;
    }

private:
    Remote r_;
};

class ForeignNorm : public Norm {
public:
    ForeignNorm(const ForeignPartHost &h, const PartSpec &s, DType dt, Device *d)
        : Norm(s, dt, d), r_(h, "norm", s, dt) {
        size_ = s.get_int("size");
    }
    void tensors(const std::string &p, TensorList &out) const override { r_.tensors(p, out); }
    void load(const std::string &p, TensorMap &t) override { r_.load(p, t); }
    size_t weight_bytes() const override { return r_.bytes(); }
    long long size() const override { return size_; }
    Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta, const int32_t *rows,
              long long n_out) override {
        // the add is the library's own; the foreign norm sees x as it is to be normalized
        if (delta) ops::add_(*ctx.dev, x, n, size_, *delta);
        long long outs = rows ? n_out : n;
        Buf out = ctx.dev->pool.get((size_t)outs * (size_t)size_ * dtype_size(out_dt));
        Json a = Json::object();
        a.set("ctx", ctx_json(ctx));
        a.set("x", addr(x));
        a.set("n", n);
        a.set("out", addr(out.ptr));
        a.set("out_dtype", dtype_name(out_dt));
        a.set("rows", addr(rows));
        a.set("n_out", outs);
        r_.ask("apply", a);
        return out;
    }

private:
    Remote r_;
    long long size_;
};

class ForeignPosition : public PositionEncoding {
public:
    ForeignPosition(const ForeignPartHost &h, const PartSpec &s, DType dt, Device *d)
        : PositionEncoding(s, dt, d), r_(h, "position", s, dt) {
        rotary_dim_ = (int)s.get_int("rotary_dim", 0);
    }
    void tensors(const std::string &p, TensorList &out) const override { r_.tensors(p, out); }
    void load(const std::string &p, TensorMap &t) override { r_.load(p, t); }
    void prepare(long long n) override {
        Json a = Json::object();
        a.set("n_positions", n);
        a.set("device", dev ? dev->index : 0);
        Json j = r_.ask("prepare", a);
        cos_ = (const float *)(uintptr_t)j.get("cos").as_uint();
        sin_ = (const float *)(uintptr_t)j.get("sin").as_uint();
        if (j.has("rotary_dim")) rotary_dim_ = (int)j.get("rotary_dim").as_int();
        n_ = j.get("n_positions").as_int();
    }
    const float *cos() const override { return cos_; }
    const float *sin() const override { return sin_; }
    int rotary_dim() const override { return rotary_dim_; }
    long long n_positions() const override { return n_; }

private:
    Remote r_;
    const float *cos_ = nullptr, *sin_ = nullptr;
    int rotary_dim_ = 0;
    long long n_ = 0;
};

}  // namespace

void register_foreign_part(const std::string &role, const std::string &kind, ForeignPartHost host) {
    if (!host.fn) fail(JB_LLM_EINVAL, "register_part: no callback");
    if (role == "mixer")
        register_part(role, kind, [host](const PartSpec &s, DType dt, Device *d) {
            return std::unique_ptr<Part>(new ForeignMixer(host, s, dt, d));
        });
    else if (role == "feed_forward")
        register_part(role, kind, [host](const PartSpec &s, DType dt, Device *d) {
            return std::unique_ptr<Part>(new ForeignFeedForward(host, s, dt, d));
        });
    else if (role == "norm")
        register_part(role, kind, [host](const PartSpec &s, DType dt, Device *d) {
            return std::unique_ptr<Part>(new ForeignNorm(host, s, dt, d));
        });
    else if (role == "position")
        register_part(role, kind, [host](const PartSpec &s, DType dt, Device *d) {
            return std::unique_ptr<Part>(new ForeignPosition(host, s, dt, d));
        });
    else
        fail(JB_LLM_EINVAL, "register_part: role '" + role + "' (mixer, feed_forward, norm, position)");
}

}  // namespace jb
