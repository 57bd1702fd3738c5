// The C interface (include/janas_b200/llm.h) over the engine.  Every function
// catches what the library throws at this boundary and turns it into a code and
// the calling thread's last-error text.
#include "api_internal.h"

#include <cstring>

using namespace jb;

namespace {

// Reads a size-prefixed struct that may be shorter (an older caller) or longer (a
// newer one) than this library's: the bytes both know are copied over the defaults.
template <class T>
T read_struct(const T *given, void (*defaults)(T *)) {
    T out;
    defaults(&out);
    if (given) {
        if (given->size < sizeof(uint32_t)) fail(JB_LLM_EINVAL, "a parameter struct's size field is not set");
        size_t n = std::min<size_t>(given->size, sizeof(T));
        memcpy(&out, given, n);
        out.size = sizeof(T);
    }
    return out;
}

GenOptions options_of(const jb_gen_options *o) {
    jb_gen_options g = read_struct<jb_gen_options>(o, jb_gen_options_default);
    if (g.n_stop < 0 || g.n_stop > JB_GEN_MAX_STOP)
        fail(JB_LLM_EINVAL, fmt("at most %d stop tokens besides eos", JB_GEN_MAX_STOP));
    GenOptions out;
    out.eos = g.eos;
    out.temperature = g.temperature;
    out.top_k = g.top_k;
    out.top_p = g.top_p;
    out.min_p = g.min_p;
    out.seed = g.seed;
    out.stop.assign(g.stop, g.stop + g.n_stop);
    out.validate();
    return out;
}

void stats_out(const GenStats &s, jb_gen_stats *st) {
    if (!st) return;
    if (st->size < sizeof(uint32_t)) fail(JB_LLM_EINVAL, "jb_gen_stats: the size field is not set");
    jb_gen_stats full;
    memset(&full, 0, sizeof full);
    full.size = st->size;
    full.prompt_tokens = s.prompt_tokens;
    full.new_tokens = s.new_tokens;
    full.passes = s.passes;
    full.forced_tokens = s.forced_tokens;
    full.batches = s.batches;
    full.prefill_seconds = s.prefill_seconds;
    full.decode_seconds = s.decode_seconds;
    full.sample_seconds = s.sample_seconds;
    full.h2d_bytes = s.h2d_bytes;
    full.d2h_bytes = s.d2h_bytes;
    memcpy(st, &full, std::min<size_t>(st->size, sizeof full));
}

jb_llm *need(jb_llm *l) {
    if (!l || !l->driver) fail(JB_LLM_EINVAL, "no open model");
    return l;
}

Engine &engine_of(jb_llm *l) {
    need(l);
    if (!l->engine) fail(JB_LLM_EINVAL, "this handle stands in for an engine; it has no device");
    return *l->engine;
}

jb_llm *wrap(std::unique_ptr<Engine> e, const jb_llm_params &p) {
    std::unique_ptr<jb_llm> l(new jb_llm());
    l->params = p;
    e->max_positions = std::min<long long>(e->max_positions, p.n_ctx);
    l->engine = std::move(e);
    l->driver = engine_driver(*l->engine);
    return l.release();
}

struct Opened {
    DType dtype;
    long long max_tokens;
    int max_seqs, device;
    jb_llm_params p;
};

Opened read_params(const jb_llm_params *given) {
    Opened o;
    o.p = read_struct<jb_llm_params>(given, jb_llm_params_default);
    if (o.p.dtype != JB_LLM_BF16 && o.p.dtype != JB_LLM_F32)
        fail(JB_LLM_EINVAL, "params.dtype: JB_LLM_BF16 or JB_LLM_F32");
    if (o.p.n_ctx == 0 || o.p.max_batch == 0) fail(JB_LLM_EINVAL, "params: n_ctx and max_batch must be positive");
    o.dtype = o.p.dtype == JB_LLM_F32 ? F32 : BF16;
    o.max_tokens = o.p.max_tokens ? (long long)o.p.max_tokens : (long long)o.p.n_ctx;
    o.max_seqs = (int)o.p.max_batch;
    o.device = o.p.device;
    return o;
}

}  // namespace

extern "C" {

int32_t jb_llm_abi_version(void) { return JB_LLM_ABI_VERSION; }
const char *jb_llm_last_error(void) { return last_error(); }

void jb_llm_params_default(jb_llm_params *p) {
    if (!p) return;
    memset(p, 0, sizeof *p);
    p->size = sizeof *p;
    p->n_ctx = 16384;       // the reference's default (include/janas/llm.h:77)
    p->max_batch = 64;
    p->dtype = JB_LLM_BF16;
    p->device = 0;
    p->max_tokens = 0;
}

void jb_gen_options_default(jb_gen_options *o) {
    if (!o) return;
    memset(o, 0, sizeof *o);
    o->size = sizeof *o;
    o->eos = -1;
}

int32_t jb_llm_open(const char *path, const jb_llm_params *p, jb_llm **out) {
    return guard([&] {
        if (!path || !out) fail(JB_LLM_EINVAL, "jb_llm_open: path and out must be given");
        *out = nullptr;
        Opened o = read_params(p);
        *out = wrap(Engine::open(path, o.dtype, o.max_tokens, o.max_seqs, o.device), o.p);
    });
}

int32_t jb_llm_open_random(const char *config_json, uint64_t seed, const jb_llm_params *p, jb_llm **out) {
    return guard([&] {
        if (!config_json || !out) fail(JB_LLM_EINVAL, "jb_llm_open_random: config_json and out must be given");
        *out = nullptr;
        Opened o = read_params(p);
        Json cfg;
        try {
            cfg = Json::parse(config_json);
        } catch (const JsonError &e) {
            fail(JB_LLM_EOPEN, std::string("config: not JSON (") + e.what() + ")");
        }
        *out = wrap(Engine::open_random(cfg, seed, o.dtype, o.max_tokens, o.max_seqs, o.device), o.p);
    });
}

int32_t jb_llm_open_spec(const char *spec_json, const char *tensors_json, uint64_t seed,
                         const jb_llm_params *p, jb_llm **out) {
    return guard([&] {
        if (!spec_json || !out) fail(JB_LLM_EINVAL, "jb_llm_open_spec: spec_json and out must be given");
        *out = nullptr;
        Opened o = read_params(p);
        ModelSpec spec = ModelSpec::from_json(Json::parse(spec_json));
        spec.validate();
        std::unique_ptr<Device> dev(new Device(o.device));
        std::unique_ptr<DecoderModel> model(new DecoderModel(spec, o.dtype, dev.get()));
        if (tensors_json && *tensors_json) {
            // the caller's tensors are copied: the model owns what it runs on
            Json ts = Json::parse(tensors_json);
            TensorMap m = tensors_from_json(*dev, ts, model->tensors(), o.dtype);
            model->load_top(m);
            for (size_t i = 0; i < model->blocks.size(); i++) model->load_layer((int)i, m);
            dev->sync();
            model->loaded = true;
        } else {
            model->load_random(seed);
        }
        *out = wrap(std::unique_ptr<Engine>(new Engine(std::move(dev), std::move(model), o.max_tokens, o.max_seqs)),
                    o.p);
    });
}

void jb_llm_close(jb_llm *llm) {
    if (!llm) return;
    guard([&] {
        if (llm->engine) {
            // a failure that the device reported stays readable after the close
            try {
                llm->engine->check_device_errors();
            } catch (const Error &e) {
                set_last_error(e.what());
            }
        }
        delete llm;
    });
}

const char *jb_llm_info(jb_llm *llm) {
    static thread_local std::string text;
    int32_t rc = guard([&] {
        need(llm);
        Json j = llm->engine ? llm->engine->describe() : Json::object();
        j.set("n_ctx", llm->driver->max_positions());
        j.set("max_batch", (long long)llm->params.max_batch);
        text = j.dump();
    });
    return rc == JB_LLM_OK ? text.c_str() : nullptr;
}

uint32_t jb_llm_n_ctx(const jb_llm *llm) {
    return llm && llm->driver ? (uint32_t)llm->driver->max_positions() : 0;
}

uint32_t jb_llm_n_vocab(const jb_llm *llm) {
    return llm && llm->driver ? (uint32_t)llm->driver->vocab_size() : 0;
}

int32_t jb_llm_check(jb_llm *llm) {
    return guard([&] { need(llm)->driver->check_errors(); });
}

// ------------------------------------------------------------------ slots, step
int32_t jb_llm_slot_new(jb_llm *llm, int32_t *slot) {
    return guard([&] {
        if (!slot) fail(JB_LLM_EINVAL, "jb_llm_slot_new: slot must be given");
        *slot = need(llm)->driver->new_sequence();
    });
}

int32_t jb_llm_slot_free(jb_llm *llm, int32_t slot) {
    return guard([&] { need(llm)->driver->free_sequence(slot); });
}

int32_t jb_llm_slot_length(jb_llm *llm, int32_t slot, uint32_t *n) {
    return guard([&] {
        long long v = need(llm)->driver->length(slot);
        if (n) *n = (uint32_t)v;
    });
}

int32_t jb_llm_slot_truncate(jb_llm *llm, int32_t slot, uint32_t n) {
    return guard([&] {
        if (!need(llm)->driver->truncate_sequence(slot, n))
            fail(JB_LLM_EINVAL, fmt("slot %d cannot go back to %u tokens", slot, n));
    });
}

int32_t jb_llm_step(jb_llm *llm, const jb_llm_piece *pieces, uint32_t np, float *logits_out,
                    uint64_t logits_cap) {
    return guard([&] {
        Engine &e = engine_of(llm);
        if (!pieces || np == 0) fail(JB_LLM_EINVAL, "a step needs at least one piece");
        std::vector<StepEntry> es;
        unsigned long long wanted = 0;
        for (uint32_t i = 0; i < np; i++) {
            es.push_back(StepEntry{pieces[i].slot, pieces[i].tokens, pieces[i].n, pieces[i].want,
                                   pieces[i].n_want});
            if (pieces[i].n_want && !pieces[i].want) fail(JB_LLM_EINVAL, "a piece wants places but names none");
            wanted += pieces[i].n_want;
        }
        unsigned long long floats = wanted * (unsigned long long)e.model->spec.vocab_size;
        if (wanted && (!logits_out || logits_cap < floats))
            fail(JB_LLM_ESMALL, fmt("the step's logits are %llu floats, the buffer holds %llu", floats,
                                    (unsigned long long)logits_cap));
        long long nw = 0;
        Buf logits = e.step(es, &nw);
        if (nw > 0)
            cuda_check(cudaMemcpyAsync(logits_out, logits.ptr, (size_t)floats * 4, cudaMemcpyDefault,
                                       e.dev->stream), "copying the logits out");
        e.dev->sync();
    });
}

// ------------------------------------------------------------------ generation
int32_t jb_llm_generate_batch(jb_llm *llm, uint32_t n, const int32_t *const *prompts,
                              const uint32_t *n_prompt, const uint32_t *max_new,
                              const jb_gen_options *const *opts, int32_t *out, uint32_t *n_out,
                              int32_t *finish, jb_gen_stats *st) {
    return guard([&] {
        need(llm);
        if (n && (!prompts || !n_prompt || !max_new || !n_out))
            fail(JB_LLM_EINVAL, "jb_llm_generate_batch: prompts, n_prompt, max_new and n_out must be given");
        std::vector<Request> reqs(n);
        unsigned long long total = 0;
        for (uint32_t i = 0; i < n; i++) {
            if (n_prompt[i] && !prompts[i]) fail(JB_LLM_EINVAL, fmt("request %u: no prompt", i));
            reqs[i].prompt.assign(prompts[i], prompts[i] + n_prompt[i]);
            reqs[i].max_new = max_new[i];
            reqs[i].options = options_of(opts ? opts[i] : nullptr);
            total += max_new[i];
        }
        if (total && !out) fail(JB_LLM_EINVAL, "jb_llm_generate_batch: out must be given");
        GenStats gs;
        std::vector<Result> res = generate(*llm->driver, reqs, (int)llm->params.max_batch, &gs);
        size_t at = 0;
        for (uint32_t i = 0; i < n; i++) {
            n_out[i] = (uint32_t)res[i].tokens.size();
            if (!res[i].tokens.empty()) memcpy(out + at, res[i].tokens.data(), res[i].tokens.size() * 4);
            if (finish) finish[i] = res[i].finish;
            at += max_new[i];
        }
        stats_out(gs, st);
    });
}

int32_t jb_llm_generate(jb_llm *llm, const int32_t *prompt, uint32_t n_prompt, uint32_t max_new,
                        const jb_gen_options *o, int32_t *out, uint32_t *n_out, int32_t *finish,
                        jb_gen_stats *st) {
    uint32_t n = 0;
    const jb_gen_options *opts[1] = {o};
    int32_t rc = jb_llm_generate_batch(llm, 1, &prompt, &n_prompt, &max_new, opts, out, &n, finish, st);
    if (n_out) *n_out = n;
    return rc;
}

// -------------------------------------------------------------------- sessions
int32_t jb_llm_session_create(jb_llm *llm, const jb_gen_options *o, jb_llm_session **out) {
    return guard([&] {
        if (!out) fail(JB_LLM_EINVAL, "jb_llm_session_create: out must be given");
        *out = nullptr;
        need(llm);
        GenOptions go = options_of(o);
        std::unique_ptr<jb_llm_session> s(new jb_llm_session());
        s->llm = llm;
        s->session.reset(new Session(*llm->driver, go));
        *out = s.release();
    });
}

void jb_llm_session_destroy(jb_llm_session *s) {
    if (!s) return;
    guard([&] { delete s; });
}

static Session &sess(jb_llm_session *s) {
    if (!s || !s->session) fail(JB_LLM_EINVAL, "no session");
    return *s->session;
}

int32_t jb_llm_session_set_options(jb_llm_session *s, const jb_gen_options *o) {
    return guard([&] { sess(s).set_options(options_of(o)); });
}

int32_t jb_llm_session_append(jb_llm_session *s, const int32_t *tokens, uint32_t n) {
    return guard([&] {
        if (n && !tokens) fail(JB_LLM_EINVAL, "jb_llm_session_append: no tokens");
        sess(s).append(tokens, n);
    });
}

int32_t jb_llm_session_prefill(jb_llm_session *s) {
    return guard([&] { sess(s).prefill(); });
}

int32_t jb_llm_session_next(jb_llm_session *s, int32_t *token) {
    int status = 0;
    int32_t rc = guard([&] {
        int32_t t = -1;
        status = sess(s).next(&t);
        if (token) *token = t;
    });
    return rc != JB_LLM_OK ? rc : status ? JB_LLM_DONE : JB_LLM_OK;
}

int32_t jb_llm_sessions_step(jb_llm_session **ss, int32_t n, int32_t *tokens, int32_t *status) {
    return guard([&] {
        if (n <= 0 || !ss || !tokens || !status) fail(JB_LLM_EINVAL, "jb_llm_sessions_step: nothing to step");
        std::vector<Session *> v;
        for (int32_t i = 0; i < n; i++) v.push_back(&sess(ss[i]));
        std::vector<int> st((size_t)n, 0);
        sessions_step(v[0]->driver, v, tokens, st.data());
        for (int32_t i = 0; i < n; i++) status[i] = st[(size_t)i];
    });
}

uint32_t jb_llm_session_computed(const jb_llm_session *s) {
    uint32_t v = 0;
    guard([&] { v = (uint32_t)sess(const_cast<jb_llm_session *>(s)).computed(); });
    return v;
}

uint32_t jb_llm_session_length(const jb_llm_session *s) {
    return s && s->session ? (uint32_t)s->session->length() : 0;
}

uint32_t jb_llm_session_tokens(const jb_llm_session *s, const int32_t **tokens) {
    if (!s || !s->session) return 0;
    if (tokens) *tokens = s->session->hist.data();
    return (uint32_t)s->session->hist.size();
}

int32_t jb_llm_session_truncate(jb_llm_session *s, uint32_t n) {
    return guard([&] { sess(s).truncate(n); });
}

int32_t jb_llm_session_reset(jb_llm_session *s) {
    return guard([&] { sess(s).reset(); });
}

int32_t jb_llm_session_stats(const jb_llm_session *s, jb_gen_stats *st) {
    return guard([&] { stats_out(sess(const_cast<jb_llm_session *>(s)).stats, st); });
}

// ---------------------------------------------------------------- decode steps
int32_t jb_llm_slot_sampler(jb_llm *llm, int32_t slot, const jb_gen_options *o) {
    return guard([&] { need(llm)->driver->set_samplers({slot}, {options_of(o).sampler()}); });
}

int32_t jb_llm_decode_begin(jb_llm *llm, const int32_t *slots, uint32_t n, const int32_t *tokens,
                            int32_t sampled, void **pending) {
    return guard([&] {
        Engine &e = engine_of(llm);
        if (!slots || n == 0 || !pending) fail(JB_LLM_EINVAL, "jb_llm_decode_begin: slots and pending must be given");
        std::vector<int> sl(slots, slots + n);
        *pending = e.decode_begin(sl, tokens, sampled != 0, false);
    });
}

int32_t jb_llm_decode_end(jb_llm *llm, void *pending, int32_t *out) {
    return guard([&] {
        Engine &e = engine_of(llm);
        if (!pending) fail(JB_LLM_EINVAL, "jb_llm_decode_end: no step");
        const std::vector<int32_t> &t = e.decode_end((PendingDecode *)pending);
        if (out) memcpy(out, t.data(), t.size() * 4);
    });
}

void *jb_llm_stream(jb_llm *llm) { return llm && llm->engine ? (void *)llm->engine->dev->stream : nullptr; }

int32_t jb_register_part(const char *role, const char *kind, jb_part_callback fn, void *user) {
    return guard([&] {
        if (!role || !kind || !fn) fail(JB_LLM_EINVAL, "jb_register_part: role, kind and fn must be given");
        register_foreign_part(role, kind, ForeignPartHost{fn, user});
    });
}

}  // extern "C"
