// jb_call: the library's other objects by name, for tools and tests.  A method name
// and JSON arguments in, JSON text out.  Device and host memory is passed as
// addresses (whole numbers).  Objects made here (caches, pools, single parts) are
// named by the id that their "new" / "build" method returns.
//
//   config.parse      {config}                       -> {architecture, config, spec, eos_token_ids}
//   config.from_dir   {dir}                          -> the same
//   config.known      {}                             -> {architectures}
//   spec.validate     {spec}
//   spec.tensors      {spec}                         -> {tensors: [{name, shape, kind, optional}]}
//   parts.registered  {role}                         -> {kinds}
//   checkpoint.list   {dir}                          -> {tensors: [{name, dtype, shape}]}
//   weights.check     {dir, tensors}                 a mismatch: code JB_LLM_EOPEN, result {missing, unexpected, wrong_shape, wrong_type}
//   weights.resident  {stored, kind, compute}        -> {dtype}
//   weights.read      {dir, name, dtype, out}        the tensor, converted to dtype, into host memory at out
//   pagepool.new {n} / slotpool.new {n}              -> {id};   pool.op {id, op, ...};   pool.free {id}
//   cache.new         {kv_specs, state_specs, max_tokens, max_seqs, dtype, device}   -> {id}   (device -1: bookkeeping only)
//   cache.op          {id | llm, op, ...}            (the ops are in cache_op below);   cache.free {id}
//   part.build        {role, spec, dtype, device}    -> {id};   part.free {id}
//   part.tensors {id, prefix}, part.load {id, prefix, tensors}, part.info {id}, part.prepare {id, n_positions},
//   part.kv_spec {id}, part.state_spec {id}, part.supports {id, kind}
//   part.apply        {id, x, n, out_dtype, delta, rows}      a norm; the result is kept: part.result {id, out}
//   part.forward      {id, ctx, h, cache}            a mixer or feed-forward -> {S, n, m}; then part.result
//   gen.tokens_needed, gen.plan_batches, gen.finish_reason, gen.goes_on     the generation loop's decisions
//   llm.open_foreign  {fn, user, max_batch}          -> {llm}: a handle whose engine is the callback fn
//   llm.set           {llm, use_graphs, max_graphs, drop_graphs, trim}   switches of an open engine -> {use_graphs, graphs}
//   llm.step_trace    {llm, entries: [{slot, tokens}]}   one step; -> {n_rows, hidden, layers}: the residual stream after every layer
//   llm.launches      {}                             -> {launches}: kernels launched so far
//   kernels.wait_selftest {limit_cycles}             -> {code}: a bounded wait that nothing ends (csrc/selftest.cu)
#include <cstring>
#include <mutex>

#include "../csrc/kernels.h"
#include "api_internal.h"

using namespace jb;

namespace {

struct PartHandle {
    std::string role;
    std::shared_ptr<Device> dev;
    std::unique_ptr<Part> part;
    Buf result;
    long long S = 0, n = 0, m = 0;
    DType result_dt = F32;
};

struct Objects {
    std::mutex mu;
    long long next = 1;
    std::map<long long, std::shared_ptr<Cache>> caches;
    std::map<long long, std::shared_ptr<PagePool>> page_pools;
    std::map<long long, std::shared_ptr<SlotPool>> slot_pools;
    std::map<long long, std::shared_ptr<PartHandle>> parts;
    std::map<int, std::shared_ptr<Device>> devices;
};

Objects &objects() {
    static Objects *o = new Objects();
    return *o;
}

std::shared_ptr<Device> device(int index) {
    Objects &o = objects();
    std::lock_guard<std::mutex> lock(o.mu);
    auto it = o.devices.find(index);
    if (it != o.devices.end()) return it->second;
    std::shared_ptr<Device> d(new Device(index));
    o.devices[index] = d;
    return d;
}

template <class T>
std::shared_ptr<T> find(std::map<long long, std::shared_ptr<T>> &m, const Json &a, const char *what) {
    Objects &o = objects();
    std::lock_guard<std::mutex> lock(o.mu);
    auto it = m.find(a.get("id").as_int());
    if (it == m.end()) fail(JB_LLM_EINVAL, std::string("no ") + what + " with this id");
    return it->second;
}

template <class T>
long long keep(std::map<long long, std::shared_ptr<T>> &m, std::shared_ptr<T> v) {
    Objects &o = objects();
    std::lock_guard<std::mutex> lock(o.mu);
    long long id = o.next++;
    m[id] = std::move(v);
    return id;
}

template <class T> T *ptr_of(const Json &j) { return (T *)(uintptr_t)j.as_uint(); }

std::vector<int> ints(const Json &j) {
    std::vector<int> v;
    for (auto &x : j.items()) v.push_back((int)x.as_int());
    return v;
}

std::vector<long long> longs(const Json &j) {
    std::vector<long long> v;
    for (auto &x : j.items()) v.push_back(x.as_int());
    return v;
}

Json int_array(const std::vector<int> &v) {
    Json a = Json::array();
    for (int x : v) a.push(x);
    return a;
}

DType dtype_of(const Json &j, DType dflt) {
    if (!j.is_string()) return dflt;
    const std::string &s = j.as_string();
    if (s == "float32" || s == "fp32") return F32;
    if (s == "bfloat16" || s == "bf16") return BF16;
    if (s == "int32") return I32;
    if (s == "int64") return I64;
    if (s == "float16") return F16;
    fail(JB_LLM_EINVAL, "unknown dtype '" + s + "'");
}

Json ok() { return Json::object(); }

Json config_result(const ArchConfig &c) {
    Json r = Json::object();
    r.set("architecture", c.architecture());
    r.set("config", c.to_json());
    r.set("spec", c.to_model_spec().to_json());
    r.set("eos_token_ids", int_array(c.eos_token_ids()));
    return r;
}

// ------------------------------------------------------------------- cache
Json cache_op(Cache &c, const Json &a) {
    std::string op = a.get("op").as_string();
    Json r = Json::object();
    auto group = [&]() -> KVGroup & {
        long long g = a.get("group").as_int();
        if (g < 0 || g >= (long long)c.groups.size()) fail(JB_LLM_EINVAL, "no such cache group");
        return *c.groups[(size_t)g];
    };
    auto live_slot = [&]() {
        int s = (int)a.get("slot").as_int();
        if (!c.slots.live(s)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", s));
        return s;
    };
    if (op == "new_sequence") r.set("slot", c.new_sequence());
    else if (op == "free_sequence") c.free_sequence((int)a.get("slot").as_int());
    else if (op == "reserve") c.reserve(ints(a.get("slots")), longs(a.get("counts")));
    else if (op == "advance") c.advance(ints(a.get("slots")), longs(a.get("counts")));
    else if (op == "truncate") r.set("ok", c.truncate((int)a.get("slot").as_int(), a.get("n").as_int()));
    else if (op == "can_truncate") r.set("ok", c.can_truncate((int)a.get("slot").as_int(), a.get("n").as_int()));
    else if (op == "length") r.set("length", c.length(live_slot()));
    else if (op == "check") c.check();
    else if (op == "tokens_held") r.set("tokens", c.tokens_held());
    else if (op == "describe") r = c.describe();
    else if (op == "held") r.set("held", group().held(live_slot()));
    else if (op == "pages") r.set("pages", int_array(group().pages[(size_t)live_slot()]));
    else if (op == "n_free_pages") r.set("n", group().pool.n_free());
    else if (op == "block_table") {
        KVGroup &g = group();
        std::vector<int> sl = ints(a.get("slots"));
        for (int s : sl)
            if (!c.slots.live(s)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", s));
        int w = c.table_width(g, sl);
        std::vector<int32_t> t(sl.size() * (size_t)w);
        c.block_table(g, sl, w, t.data());
        Json rows = Json::array();
        for (size_t i = 0; i < sl.size(); i++) {
            Json row = Json::array();
            for (int j = 0; j < w; j++) row.push((int)t[i * (size_t)w + (size_t)j]);
            rows.push(row);
        }
        r.set("table", rows);
        r.set("width", w);
    } else if (op == "set_samplers") {
        std::vector<SamplerSettings> ss;
        for (auto &s : a.get("settings").items())
            ss.push_back(SamplerSettings{s.get("seed").as_uint(), (float)s.get("temperature").as_double(),
                                         (int)s.get("top_k").as_int(), (float)s.get("top_p").as_double(),
                                         (float)s.get("min_p").as_double()});
        c.set_samplers(ints(a.get("slots")), ss);
        if (c.dev) c.dev->sync();
    } else if (op == "state") {
        int e = (int)a.get("entry").as_int();
        auto it = c.mixer_state.find(e);
        if (it == c.mixer_state.end()) fail(JB_LLM_EINVAL, "this entry keeps no state");
        r.set("ptr", (unsigned long long)(uintptr_t)it->second.ptr);
        Json sh = Json::array();
        for (auto s : it->second.shape) sh.push(s);
        r.set("shape", sh);
        r.set("dtype", dtype_name(it->second.dt));
    } else {
        fail(JB_LLM_EINVAL, "cache.op: no op '" + op + "'");
    }
    return r;
}

// ------------------------------------------------------------------- parts
StepContext ctx_from_json(const Json &j, Device *dev) {
    StepContext c;
    std::string kind = j.get("kind").is_string() ? j.get("kind").as_string() : "prefill";
    c.kind = kind == "decode" ? DECODE : kind == "extend" ? EXTEND : PREFILL;
    c.dtype = dtype_of(j.get("dtype"), F32);
    c.dev = dev;
    c.n_rows = j.get("n_rows").as_int();
    c.n_seqs = (int)j.get("n_seqs").as_int();
    c.hidden = j.get("hidden").as_int();
    c.row_pos = ptr_of<const int32_t>(j.get("row_pos"));
    c.row_seq = ptr_of<const int32_t>(j.get("row_seq"));
    c.seq_slot = ptr_of<const int32_t>(j.get("seq_slot"));
    c.seq_slots = ints(j.get("seq_slots"));
    c.seq_pos0 = longs(j.get("seq_pos0"));
    c.seq_len = longs(j.get("seq_len"));
    c.seq_row0 = longs(j.get("seq_row0"));
    c.max_pos = j.get("max_pos").as_int();
    return c;
}

LayerCache cache_from_json(const Json &j) {
    LayerCache c;
    if (!j.is_object()) return c;
    c.kv.k = ptr_of<void>(j.get("k"));
    c.kv.v = ptr_of<void>(j.get("v"));
    c.kv.n_pages = j.get("n_pages").as_int();
    c.kv.dt = dtype_of(j.get("dtype"), F32);
    c.kv.block_table = ptr_of<const int32_t>(j.get("block_table"));
    c.kv.bt_stride = (int)j.get("bt_stride").as_int();
    c.kv.writes = j.has("writes") ? j.get("writes").as_bool() : true;
    c.kv_heads = (int)j.get("kv_heads").as_int();
    c.head_dim = (int)j.get("head_dim").as_int();
    c.state = ptr_of<void>(j.get("state"));
    c.state_spec.shape = longs(j.get("state_shape"));
    c.state_spec.dtype = dtype_of(j.get("state_dtype"), F32);
    c.n_slots = (int)j.get("n_slots").as_int();
    return c;
}

Json part_call(const std::string &method, const Json &a) {
    Objects &o = objects();
    if (method == "part.build") {
        std::shared_ptr<PartHandle> h(new PartHandle());
        h->role = a.get("role").as_string();
        int di = a.has("device") ? (int)a.get("device").as_int() : 0;
        if (di >= 0) h->dev = device(di);
        h->part = build_part(h->role, PartSpec::from_json(a.get("spec")), dtype_of(a.get("dtype"), F32),
                             h->dev.get());
        Json r = Json::object();
        r.set("id", keep(o.parts, h));
        return r;
    }
    std::shared_ptr<PartHandle> h = find(o.parts, a, "part");
    Part &p = *h->part;
    if (method == "part.free") {
        std::lock_guard<std::mutex> lock(o.mu);
        o.parts.erase(a.get("id").as_int());
        return ok();
    }
    if (method == "part.tensors") {
        TensorList l;
        p.tensors(a.get("prefix").as_string(), l);
        Json r = Json::object();
        r.set("tensors", tensor_list_json(l));
        return r;
    }
    if (method == "part.info") return p.info();
    if (!h->dev) fail(JB_LLM_EINVAL, "this part was built without a device");
    Device &d = *h->dev;
    d.make_current();
    if (method == "part.load") {
        TensorList l;
        std::string prefix = a.get("prefix").as_string();
        p.tensors(prefix, l);
        TensorMap m = tensors_from_json(d, a.get("tensors"), l, p.dtype);
        p.load(prefix, m);
        d.sync();
        return ok();
    }
    if (method == "part.prepare") {
        long long n = a.get("n_positions").as_int();
        if (auto *m = dynamic_cast<Mixer *>(&p)) m->prepare(n);
        else if (auto *pe = dynamic_cast<PositionEncoding *>(&p)) pe->prepare(n);
        else fail(JB_LLM_EINVAL, "this part has nothing to prepare");
        d.sync();
        return p.info();
    }
    if (method == "part.kv_spec" || method == "part.state_spec" || method == "part.supports") {
        auto *m = dynamic_cast<Mixer *>(&p);
        if (!m) fail(JB_LLM_EINVAL, "not a mixer");
        Json r = Json::object();
        if (method == "part.kv_spec") {
            KVSpec s = m->kv_spec();
            if (!s.none()) {
                r.set("num_kv_heads", s.num_kv_heads);
                r.set("head_dim", s.head_dim);
                r.set("window", s.window);
            }
        } else if (method == "part.state_spec") {
            StateSpec s = m->state_spec();
            if (!s.none()) {
                Json sh = Json::array();
                for (auto v : s.shape) sh.push(v);
                r.set("shape", sh);
                r.set("dtype", dtype_name(s.dtype));
            }
        } else {
            std::string k = a.get("kind").as_string();
            r.set("ok", m->supports(k == "decode" ? DECODE : k == "extend" ? EXTEND : PREFILL));
        }
        return r;
    }
    if (method == "part.apply") {
        auto *nm = dynamic_cast<Norm *>(&p);
        if (!nm) fail(JB_LLM_EINVAL, "not a norm");
        long long n = a.get("n").as_int();
        StepContext ctx;
        ctx.dev = &d;
        ctx.dtype = p.dtype;
        ctx.n_rows = n;
        ctx.hidden = nm->size();
        Stack delta;
        bool has_delta = a.get("delta").is_object();
        if (has_delta) {
            // the caller's partial sums are copied: a Stack owns its memory
            delta.S = (int)a.get("delta").get("S").as_int();
            delta.n = n;
            delta.m = nm->size();
            size_t bytes = (size_t)delta.S * (size_t)n * (size_t)delta.m * 4;
            delta.buf = d.pool.get(bytes);
            cuda_check(cudaMemcpyAsync(delta.buf.ptr, ptr_of<void>(a.get("delta").get("ptr")), bytes,
                                       cudaMemcpyDeviceToDevice, d.stream), "copy on the device");
        }
        const Json &rows = a.get("rows");
        long long n_out = rows.is_object() ? rows.get("n").as_int() : 0;
        DType out_dt = dtype_of(a.get("out_dtype"), F32);
        h->result = nm->apply(ctx, ptr_of<float>(a.get("x")), n, out_dt, has_delta ? &delta : nullptr,
                              rows.is_object() ? ptr_of<const int32_t>(rows.get("ptr")) : nullptr, n_out);
        d.sync();
        h->S = 1;
        h->n = rows.is_object() ? n_out : n;
        h->m = nm->size();
        h->result_dt = out_dt;
    } else if (method == "part.forward") {
        StepContext ctx = ctx_from_json(a.get("ctx"), &d);
        const void *hin = ptr_of<const void>(a.get("h"));
        Stack out;
        if (auto *m = dynamic_cast<Mixer *>(&p)) {
            LayerCache lc = cache_from_json(a.get("cache"));
            out = m->forward(ctx, hin, lc);
        } else if (auto *f = dynamic_cast<FeedForward *>(&p)) {
            out = f->forward(ctx, hin);
        } else {
            fail(JB_LLM_EINVAL, "not a mixer or a feed-forward");
        }
        d.sync();
        h->S = out.S;
        h->n = out.n;
        h->m = out.m;
        h->result = std::move(out.buf);
        h->result_dt = F32;
    } else if (method == "part.result") {
        if (!h->result) fail(JB_LLM_EINVAL, "no result is kept");
        size_t bytes = (size_t)h->S * (size_t)h->n * (size_t)h->m * dtype_size(h->result_dt);
        cuda_check(cudaMemcpyAsync(ptr_of<void>(a.get("out")), h->result.ptr, bytes, cudaMemcpyDefault, d.stream),
                   "copying a result out");
        d.sync();
        return ok();
    } else {
        fail(JB_LLM_EINVAL, "no method '" + method + "'");
    }
    Json r = Json::object();
    r.set("S", h->S);
    r.set("n", h->n);
    r.set("m", h->m);
    r.set("dtype", dtype_name(h->result_dt));
    return r;
}

// -------------------------------------------------------- a stand-in engine
class ForeignDriver : public Driver {
public:
    ForeignDriver(ForeignCall fn, void *user) : fn_(fn), user_(user) {}
    Json ask(const char *method, const Json &a = Json::object()) const {
        const char *r = fn_(user_, method, a.dump().c_str());
        if (!r) fail(JB_LLM_EFAIL, std::string("the stand-in engine failed in '") + method + "'");
        Json j = Json::parse(r);
        if (j.is_object() && j.has("error")) {
            int code = j.has("code") ? (int)j.get("code").as_int() : JB_LLM_EFAIL;
            if (code == JB_LLM_EFULL) throw CacheFull(j.get("error").as_string());
            fail(code, j.get("error").as_string());
        }
        return j;
    }
    static Json slot_arg(int slot) {
        Json a = Json::object();
        a.set("slot", slot);
        return a;
    }
    long long vocab_size() const override { return ask("vocab_size").get("value").as_int(); }
    long long max_positions() const override { return ask("max_positions").get("value").as_int(); }
    int free_slots() const override { return (int)ask("free_slots").get("value").as_int(); }
    long long free_tokens() const override { return ask("free_tokens").get("value").as_int(); }
    int new_sequence() override { return (int)ask("new_sequence").get("slot").as_int(); }
    void free_sequence(int slot) override { ask("free_sequence", slot_arg(slot)); }
    long long length(int slot) const override { return ask("length", slot_arg(slot)).get("value").as_int(); }
    bool truncate_sequence(int slot, long long n) override {
        Json a = slot_arg(slot);
        a.set("n", n);
        return ask("truncate", a).get("ok").as_bool();
    }
    void set_samplers(const std::vector<int> &slots, const std::vector<SamplerSettings> &s) override {
        Json a = Json::object();
        a.set("slots", int_array(slots));
        Json ss = Json::array();
        for (auto &x : s) {
            Json e = Json::object();
            e.set("seed", x.seed);
            e.set("temperature", (double)x.temperature);
            e.set("top_k", x.top_k);
            e.set("top_p", (double)x.top_p);
            e.set("min_p", (double)x.min_p);
            ss.push(e);
        }
        a.set("settings", ss);
        ask("set_samplers", a);
    }
    bool needs_long_way(float, int) const override { return false; }
    bool supports_extend() const override { return ask("supports_extend").get("ok").as_bool(); }
    std::vector<int32_t> run(const std::vector<FeedEntry> &entries, bool sampled, bool long_way,
                             int *forced) override {
        Json a = Json::object();
        Json es = Json::array();
        for (auto &e : entries) {
            Json j = Json::object();
            j.set("slot", e.slot);
            Json t = Json::array();
            for (long long i = 0; i < e.n; i++) t.push((int)e.tokens[i]);
            j.set("tokens", t);
            j.set("want", e.want);
            es.push(j);
        }
        a.set("entries", es);
        a.set("sampled", sampled);
        a.set("long_way", long_way);
        Json r = ask("run", a);
        if (forced) *forced = (int)r.get("forced").as_int();
        std::vector<int32_t> out;
        for (auto &t : r.get("tokens").items()) out.push_back((int32_t)t.as_int());
        return out;
    }

    bool decodes_ahead() const override { return ask("decodes_ahead").get("ok").as_bool(); }
    void *decode_begin(const std::vector<int> &slots, const int32_t *tokens, bool sampled,
                       bool long_way) override {
        Json a = Json::object();
        a.set("slots", int_array(slots));
        if (tokens) {
            Json t = Json::array();
            for (size_t i = 0; i < slots.size(); i++) t.push((int)tokens[i]);
            a.set("tokens", t);
        } else {
            a.set("tokens", Json());
        }
        a.set("sampled", sampled);
        // the stand-in names its steps by whole numbers from 1
        return (void *)(uintptr_t)ask("decode_begin", a).get("pending").as_uint();
    }
    std::vector<int32_t> decode_end(void *pending) override {
        Json a = Json::object();
        a.set("pending", (unsigned long long)(uintptr_t)pending);
        std::vector<int32_t> out;
        Json r = ask("decode_end", a);
        for (auto &t : r.get("tokens").items()) out.push_back((int32_t)t.as_int());
        return out;
    }

private:
    ForeignCall fn_;
    void *user_;
};

}  // namespace

namespace jb {

std::unique_ptr<Driver> foreign_driver(ForeignCall fn, void *user) {
    return std::unique_ptr<Driver>(new ForeignDriver(fn, user));
}

TensorMap tensors_from_json(Device &dev, const Json &tensors, const TensorList &expected, DType compute) {
    if (!tensors.is_object()) fail(JB_LLM_EINVAL, "tensors: {name: {ptr, dtype, shape}}");
    TensorMap m;
    std::vector<std::string> missing, unexpected;
    std::set<std::string> names;
    dev.make_current();
    for (auto &kv : expected) {
        names.insert(kv.first);
        const Json &t = tensors.get(kv.first);
        if (!t.is_object()) {
            if (!kv.second.optional) missing.push_back(kv.first);
            continue;
        }
        std::vector<long long> shape = longs(t.get("shape"));
        if (shape != kv.second.shape) fail(JB_LLM_EOPEN, "tensor " + kv.first + ": unexpected shape");
        DType src = dtype_of(t.get("dtype"), F32);
        if (src != F32 && src != BF16) fail(JB_LLM_EOPEN, "tensor " + kv.first + ": float32 or bfloat16 is needed");
        DType keep_as = compute == F32 ? F32 : src;
        DevTensor d = dev.tensor(keep_as, shape);
        if (jb_convert(ptr_of<const void>(t.get("ptr")), src, d.ptr, keep_as, d.numel(), dev.stream) != 0)
            fail(JB_LLM_EFAIL, "tensor " + kv.first + ": the copy could not be launched");
        m[kv.first] = d;
    }
    for (auto &kv : tensors.members())
        if (!names.count(kv.first)) unexpected.push_back(kv.first);
    if (!missing.empty() || !unexpected.empty()) {
        std::string msg = "the tensors do not match the model";
        for (auto &n : missing) msg += "\n  missing: " + n;
        for (auto &n : unexpected) msg += "\n  unexpected: " + n;
        fail(JB_LLM_EOPEN, msg);
    }
    dev.sync();
    return m;
}

}  // namespace jb

static Json dispatch(const std::string &method, const Json &a, Json *error_detail) {
    Objects &o = objects();
    Json r = Json::object();
    if (method == "config.parse") return config_result(*config_from_json(a.get("config")));
    if (method == "config.from_dir") return config_result(*config_from_dir(a.get("dir").as_string()));
    if (method == "config.known") {
        Json l = Json::array();
        for (auto &n : known_architectures()) l.push(n);
        r.set("architectures", l);
        return r;
    }
    if (method == "spec.validate") {
        ModelSpec::from_json(a.get("spec")).validate();
        return r;
    }
    if (method == "spec.tensors") {
        DecoderModel m(ModelSpec::from_json(a.get("spec")), F32, nullptr);
        r.set("tensors", tensor_list_json(m.tensors()));
        return r;
    }
    if (method == "parts.registered") {
        Json l = Json::array();
        for (auto &n : registered_parts(a.get("role").as_string())) l.push(n);
        r.set("kinds", l);
        return r;
    }
    if (method == "checkpoint.list") {
        Checkpoint c(a.get("dir").as_string());
        Json l = Json::array();
        for (auto &n : c.names) {
            const TensorInfo &t = c.tensors.at(n);
            Json e = Json::object();
            e.set("name", n);
            e.set("dtype", t.dtype);
            Json sh = Json::array();
            for (auto s : t.shape) sh.push(s);
            e.set("shape", sh);
            l.push(e);
        }
        r.set("tensors", l);
        return r;
    }
    if (method == "weights.check") {
        Checkpoint c(a.get("dir").as_string());
        try {
            check_weights(c, tensor_list_from_json(a.get("tensors")));
        } catch (const WeightMismatch &e) {
            *error_detail = e.to_json();
            throw;
        }
        return r;
    }
    if (method == "weights.resident") {
        r.set("dtype", dtype_name(resident_dtype(a.get("stored").as_string(), parse_kind(a.get("kind").as_string()),
                                                 parse_compute_dtype(a.get("compute").as_string()))));
        return r;
    }
    if (method == "weights.read") {
        Checkpoint c(a.get("dir").as_string());
        auto it = c.tensors.find(a.get("name").as_string());
        if (it == c.tensors.end()) fail(JB_LLM_EOPEN, "tensor " + a.get("name").as_string() + " is missing");
        convert_tensor(it->second, dtype_of(a.get("dtype"), F32), ptr_of<void>(a.get("out")));
        return r;
    }
    if (method == "pagepool.new") {
        r.set("id", keep(o.page_pools, std::make_shared<PagePool>((int)a.get("n").as_int(), "cache")));
        return r;
    }
    if (method == "slotpool.new") {
        r.set("id", keep(o.slot_pools, std::make_shared<SlotPool>((int)a.get("n").as_int())));
        return r;
    }
    if (method == "pool.free") {
        std::lock_guard<std::mutex> lock(o.mu);
        o.page_pools.erase(a.get("id").as_int());
        o.slot_pools.erase(a.get("id").as_int());
        return r;
    }
    if (method == "pool.op") {
        std::string op = a.get("op").as_string();
        long long id = a.get("id").as_int();
        std::shared_ptr<PagePool> pp;
        std::shared_ptr<SlotPool> sp;
        {
            std::lock_guard<std::mutex> lock(o.mu);
            if (o.page_pools.count(id)) pp = o.page_pools[id];
            if (o.slot_pools.count(id)) sp = o.slot_pools[id];
        }
        if (pp) {
            if (op == "take") r.set("pages", int_array(pp->take((int)a.get("count").as_int())));
            else if (op == "give_back") pp->give_back(ints(a.get("pages")));
            else if (op == "check") pp->check();
            else if (op == "n_free") r.set("n", pp->n_free());
            else fail(JB_LLM_EINVAL, "pool.op: no op '" + op + "'");
        } else if (sp) {
            if (op == "take") r.set("slot", sp->take());
            else if (op == "give_back") sp->give_back((int)a.get("slot").as_int());
            else if (op == "live") r.set("ok", sp->live((int)a.get("slot").as_int()));
            else if (op == "check") sp->check();
            else if (op == "n_free") r.set("n", sp->n_free());
            else fail(JB_LLM_EINVAL, "pool.op: no op '" + op + "'");
        } else {
            fail(JB_LLM_EINVAL, "no pool with this id");
        }
        return r;
    }
    if (method == "cache.new") {
        std::vector<KVSpec> kv;
        for (auto &s : a.get("kv_specs").items())
            kv.push_back(s.is_object() ? KVSpec{(int)s.get("num_kv_heads").as_int(), (int)s.get("head_dim").as_int(),
                                                (int)s.get("window").as_int()}
                                       : KVSpec());
        std::vector<StateSpec> st;
        for (auto &s : a.get("state_specs").items()) {
            StateSpec sp;
            if (s.is_object()) {
                sp.shape = longs(s.get("shape"));
                sp.dtype = dtype_of(s.get("dtype"), F32);
            }
            st.push_back(sp);
        }
        int di = a.has("device") ? (int)a.get("device").as_int() : -1;
        std::shared_ptr<Device> dev = di >= 0 ? device(di) : nullptr;
        // the cache keeps its device alive through the objects table
        std::shared_ptr<Cache> c(new Cache(kv, st, a.get("max_tokens").as_int(), (int)a.get("max_seqs").as_int(),
                                           dtype_of(a.get("dtype"), F32), dev.get()));
        r.set("id", keep(o.caches, c));
        return r;
    }
    if (method == "cache.free") {
        std::lock_guard<std::mutex> lock(o.mu);
        o.caches.erase(a.get("id").as_int());
        return r;
    }
    if (method == "cache.op") {
        if (a.has("llm")) {
            jb_llm *l = ptr_of<jb_llm>(a.get("llm"));
            if (!l || !l->engine) fail(JB_LLM_EINVAL, "cache.op: no engine behind this handle");
            l->engine->dev->make_current();
            return cache_op(*l->engine->cache, a);
        }
        std::shared_ptr<Cache> c = find(o.caches, a, "cache");
        if (c->dev) c->dev->make_current();
        return cache_op(*c, a);
    }
    if (method.compare(0, 5, "part.") == 0) return part_call(method, a);
    if (method == "gen.tokens_needed") {
        r.set("tokens", tokens_needed(a.get("prompt_len").as_int(), a.get("max_new").as_int(),
                                      a.get("max_positions").as_int()));
        return r;
    }
    if (method == "gen.plan_batches") {
        auto plan = plan_batches(longs(a.get("prompt_lens")), longs(a.get("max_news")), (int)a.get("max_batch").as_int(),
                                 a.get("max_tokens").as_int(), a.get("max_positions").as_int());
        Json l = Json::array();
        for (auto &b : plan) l.push(int_array(b));
        r.set("batches", l);
        return r;
    }
    if (method == "gen.finish_reason") {
        GenOptions go;
        go.eos = a.has("eos") ? (int)a.get("eos").as_int() : -1;
        go.stop = ints(a.get("stop"));
        int f = finish_reason((int)a.get("token").as_int(), a.get("n_generated").as_int(), a.get("max_new").as_int(),
                              a.get("length").as_int(), a.get("max_positions").as_int(), go);
        r.set("finish", f == FINISH_NONE ? Json() : Json(finish_name(f)));
        return r;
    }
    if (method == "gen.goes_on") {
        r.set("ok", goes_on_unless_stopped(a.get("n_generated").as_int(), a.get("max_new").as_int(),
                                           a.get("length").as_int(), a.get("max_positions").as_int()));
        return r;
    }
    if (method == "llm.open_foreign") {
        ForeignCall fn = (ForeignCall)(uintptr_t)a.get("fn").as_uint();
        if (!fn) fail(JB_LLM_EINVAL, "llm.open_foreign: no callback");
        std::unique_ptr<jb_llm> l(new jb_llm());
        jb_llm_params_default(&l->params);
        if (a.has("max_batch")) l->params.max_batch = (uint32_t)a.get("max_batch").as_int();
        l->driver = foreign_driver(fn, ptr_of<void>(a.get("user")));
        r.set("llm", (unsigned long long)(uintptr_t)l.release());
        return r;
    }
    if (method == "llm.set") {
        jb_llm *l = ptr_of<jb_llm>(a.get("llm"));
        if (!l || !l->engine) fail(JB_LLM_EINVAL, "llm.set: no engine behind this handle");
        Engine &e = *l->engine;
        if (a.has("use_graphs")) e.use_graphs = a.get("use_graphs").as_bool() && e.model->graph_safe();
        if (a.has("max_graphs")) e.max_graphs = (size_t)std::max<long long>(1, a.get("max_graphs").as_int());
        if (a.get("drop_graphs").as_bool()) e.drop_graphs();
        if (a.get("trim").as_bool()) {
            e.dev->sync();
            e.dev->pool.trim();
        }
        r.set("use_graphs", e.use_graphs);
        r.set("graphs", (long long)e.n_graphs());
        return r;
    }
    if (method == "llm.step_trace") {
        // {llm, entries: [{slot, tokens}]} -> {n_rows, hidden, layers: [[n_rows * hidden floats] per entry of
        // the run order]}: one step whose residual stream is copied out after every layer
        jb_llm *l = ptr_of<jb_llm>(a.get("llm"));
        if (!l || !l->engine) fail(JB_LLM_EINVAL, "llm.step_trace: no engine behind this handle");
        Engine &e = *l->engine;
        std::vector<StepEntry> entries;
        std::vector<std::vector<int32_t>> toks;
        for (const Json &je : a.get("entries").items()) {
            toks.emplace_back();
            for (const Json &t : je.get("tokens").items()) toks.back().push_back((int32_t)t.as_int());
        }
        size_t i = 0;
        long long rows = 0;
        for (const Json &je : a.get("entries").items()) {
            StepEntry se;
            se.slot = (int)je.get("slot").as_int();
            se.tokens = toks[i].data();
            se.n = (long long)toks[i].size();
            rows += se.n;
            entries.push_back(se);
            i++;
        }
        std::vector<std::vector<float>> layers;
        e.trace = &layers;
        try {
            long long n_wanted = 0;
            e.step(entries, &n_wanted);
            e.dev->sync();
        } catch (...) {
            e.trace = nullptr;
            throw;
        }
        e.trace = nullptr;
        Json out = Json::array();
        for (auto &v : layers) {
            Json row = Json::array();
            for (float f : v) row.push((double)f);
            out.push(std::move(row));
        }
        r.set("n_rows", rows);
        r.set("hidden", e.model->spec.hidden_size);
        r.set("layers", std::move(out));
        return r;
    }
    if (method == "llm.launches") {
        r.set("launches", ops::launches());
        return r;
    }
    if (method == "kernels.wait_selftest") {
        r.set("code", jb_wait_selftest(a.get("limit_cycles").as_int()));
        return r;
    }
    fail(JB_LLM_EINVAL, "no method '" + method + "'");
}

extern "C" void jb_free(char *text) { free(text); }

// The result is the caller's (jb_free), not a buffer of the library's that the next
// call would write over: a caller's finalizers may call in here between a call's
// return and the reading of its result.
extern "C" int32_t jb_call(const char *method, const char *args_json, char **result) {
    std::string text;
    Json detail;
    int32_t rc = guard([&] {
        if (!method) fail(JB_LLM_EINVAL, "jb_call: no method");
        Json a = args_json && *args_json ? Json::parse(args_json) : Json::object();
        text = dispatch(method, a, &detail).dump();
    });
    if (rc != JB_LLM_OK) text = detail.is_null() ? "{}" : detail.dump();
    if (result) {
        *result = (char *)malloc(text.size() + 1);
        if (!*result) return JB_LLM_ENOMEM;
        memcpy(*result, text.c_str(), text.size() + 1);
    }
    return rc;
}
