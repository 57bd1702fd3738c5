#include "engine.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <set>

#include "../csrc/kernels.h"
#include "graph.h"

namespace jb {

const std::vector<int32_t> &PendingDecode::result() {
    if (!taken) {
        if (event) {
            cuda_check(cudaEventSynchronize(event), "waiting for a decode step");
            tokens.assign(out_host, out_host + n);
        }
        taken = true;
    }
    return tokens;
}

Engine::Engine(std::unique_ptr<Device> d, std::unique_ptr<DecoderModel> m, long long max_tokens,
               int max_seqs)
    : dev(std::move(d)), model(std::move(m)), dtype(model->dtype) {
    if (!dev) fail(JB_LLM_EFAIL, "janas_b200 runs on a CUDA device only; there is no CPU path");
    if (jb_page() != PAGE)
        fail(JB_LLM_EFAIL, fmt("the kernels were built for pages of %d positions, the cache for %d",
                               jb_page(), PAGE));
    if (max_tokens <= 0) fail(JB_LLM_EINVAL, "max_tokens must be positive");
    if (max_seqs <= 0) max_seqs = (int)std::max(1ll, std::min(256ll, (max_tokens + 63) / 64));
    dev->make_current();
    cache.reset(new Cache(model->kv_specs(), model->state_specs(), max_tokens, max_seqs, dtype, dev.get()));
    max_positions = std::min(model->spec.max_positions, cache->max_tokens);
    model->prepare(max_positions);
    const char *env = getenv("JANAS_B200_GRAPHS");
    use_graphs = !(env && strcmp(env, "0") == 0) && model->graph_safe();
    for (size_t e = 0; e < model->spec.run_order.size(); e++) {
        int src = model->spec.run_order[e].cache_of >= 0 ? model->spec.run_order[e].cache_of : (int)e;
        cache_entry_.push_back(cache->group_of.count(src) ? src : -1);
    }
    // a pool that gives memory back must first let go of the graphs that hold its addresses
    dev->pool.before_trim = [this] { drop_graphs(); };
}

Engine::~Engine() {
    if (dev) {
        cudaStreamSynchronize(dev->stream);
        dev->pool.before_trim = nullptr;
    }
    graphs_.clear();
}

static std::unique_ptr<Engine> make_engine(std::unique_ptr<ArchConfig> cfg, DType dtype, long long max_tokens,
                                           int max_seqs, int device, const Checkpoint *ckpt,
                                           unsigned long long seed) {
    ModelSpec spec = cfg->to_model_spec();
    // the configuration and the folder are read and checked before the device is touched
    if (ckpt) {
        DecoderModel dry(spec, dtype, nullptr);
        check_weights(*ckpt, dry.tensors());
    }
    std::unique_ptr<Device> dev(new Device(device));
    std::unique_ptr<DecoderModel> model(new DecoderModel(spec, dtype, dev.get()));
    if (ckpt) model->load_checkpoint(*ckpt);
    else model->load_random(seed);
    std::unique_ptr<Engine> eng(new Engine(std::move(dev), std::move(model), max_tokens, max_seqs));
    eng->config = std::move(cfg);
    return eng;
}

std::unique_ptr<Engine> Engine::open(const std::string &model_dir, DType dtype, long long max_tokens,
                                     int max_seqs, int device) {
    std::unique_ptr<ArchConfig> cfg = config_from_dir(model_dir);
    Checkpoint ckpt(model_dir);
    return make_engine(std::move(cfg), dtype, max_tokens, max_seqs, device, &ckpt, 0);
}

std::unique_ptr<Engine> Engine::open_random(const Json &config_json, unsigned long long seed, DType dtype,
                                            long long max_tokens, int max_seqs, int device) {
    return make_engine(config_from_json(config_json), dtype, max_tokens, max_seqs, device, nullptr, seed);
}

// ------------------------------------------------------------- sequences
void Engine::free_sequence(int slot) {
    cache->free_sequence(slot);
    if (std::find(last_slots_.begin(), last_slots_.end(), slot) != last_slots_.end()) {
        last_graph_ = nullptr;      // no step can go on from that step's tokens any more
        last_slots_.clear();
    }
}

long long Engine::length(int slot) const {
    if (!cache->slots.live(slot)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", slot));
    return cache->length(slot);
}

bool Engine::truncate_sequence(int slot, long long n) {
    if (!cache->truncate(slot, n)) return false;
    if (std::find(last_slots_.begin(), last_slots_.end(), slot) != last_slots_.end()) {
        last_graph_ = nullptr;
        last_slots_.clear();
    }
    return true;
}

// ------------------------------------------------------------------ step
Engine::Plan Engine::plan(const std::vector<StepEntry> &entries) const {
    if (entries.empty()) fail(JB_LLM_EINVAL, "a step needs at least one sequence");
    long long vocab = model->spec.vocab_size;
    Plan p;
    std::set<int> seen;
    bool all_start = true, all_one = true;
    for (auto &ent : entries) {
        if (!cache->slots.live(ent.slot)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", ent.slot));
        if (!seen.insert(ent.slot).second) fail(JB_LLM_EINVAL, fmt("slot %d appears twice in one step", ent.slot));
        if (ent.n <= 0 || !ent.tokens) fail(JB_LLM_EINVAL, fmt("slot %d: no tokens", ent.slot));
        long long p0 = cache->length(ent.slot);
        if (p0 + ent.n > max_positions)
            fail(JB_LLM_EFULL, fmt("slot %d: %lld + %lld tokens exceed the %lld positions of the context",
                                   ent.slot, p0, ent.n, max_positions));
        for (long long i = 0; i < ent.n_want; i++)
            if (ent.want[i] < 0 || ent.want[i] >= ent.n)
                fail(JB_LLM_EINVAL, fmt("slot %d: wanted place %d is not among its %lld tokens", ent.slot,
                                        ent.want[i], ent.n));
        for (long long i = 0; i < ent.n; i++)
            if (ent.tokens[i] < 0 || ent.tokens[i] >= vocab)
                fail(JB_LLM_EINVAL, fmt("a token id lies outside the vocabulary of %lld", vocab));
        p.slots.push_back(ent.slot);
        p.pos0.push_back(p0);
        p.lens.push_back(ent.n);
        p.tokens.insert(p.tokens.end(), ent.tokens, ent.tokens + ent.n);
        p.n_rows += ent.n;
        p.n_want += ent.n_want;
        all_start = all_start && p0 == 0;
        all_one = all_one && ent.n == 1;
    }
    if (p.n_rows > 0x7fffffffll) fail(JB_LLM_EINVAL, "too many tokens for one step");
    p.kind = all_start ? PREFILL : all_one ? DECODE : EXTEND;
    if (!model->supports(p.kind))
        fail(JB_LLM_EINVAL, "this model cannot append several tokens at once to sequences that already "
                            "hold some (a mixer does not support it)");
    return p;
}

std::vector<LayerCache> Engine::layer_caches(
    const std::map<const KVGroup *, std::pair<const int32_t *, int>> &bt) {
    std::vector<LayerCache> out;
    for (size_t e = 0; e < model->spec.run_order.size(); e++) {
        LayerCache lc;
        lc.kv.writes = model->spec.run_order[e].cache_of < 0;
        auto st = cache->mixer_state.find((int)e);
        if (st != cache->mixer_state.end()) {
            lc.state = st->second.ptr;
            lc.state_spec = cache->state_spec[(int)e];
        }
        lc.n_slots = cache->max_seqs;
        int src = cache_entry_[e];
        if (src >= 0) {
            KVGroup *g = cache->group_of[src];
            lc.kv.k = g->k_of(src);
            lc.kv.v = g->v_of(src);
            lc.kv.n_pages = g->pool.n_pages();
            lc.kv.dt = cache->dtype;
            auto it = bt.find(g);
            lc.kv.block_table = it->second.first;
            lc.kv.bt_stride = it->second.second;
            lc.kv_heads = g->spec.num_kv_heads;
            lc.head_dim = g->spec.head_dim;
        }
        out.push_back(lc);
    }
    return out;
}

Buf Engine::step(const std::vector<StepEntry> &entries, long long *n_wanted) {
    Plan p = plan(entries);
    dev->make_current();
    cache->reserve(p.slots, p.lens);     // CacheFull leaves everything as it was

    long long n = p.n_rows;
    size_t B = entries.size();
    std::vector<long long> row0(B + 1, 0);
    for (size_t i = 0; i < B; i++) row0[i + 1] = row0[i] + p.lens[i];
    bool all_rows = p.n_want == n;
    {
        long long r = 0;
        for (size_t i = 0; i < B && all_rows; i++)
            for (long long w = 0; w < entries[i].n_want && all_rows; w++, r++)
                all_rows = row0[i] + entries[i].want[w] == r;
    }

    // one host buffer, one copy: tokens | row_pos | row_seq | slots | want | block tables
    std::vector<int> widths;
    size_t total = (size_t)n * 3 + B + (size_t)p.n_want;
    for (auto &g : cache->groups) {
        widths.push_back(cache->table_width(*g, p.slots));
        total += B * (size_t)widths.back();
    }
    int32_t *h = (int32_t *)dev->pinned(total * 4);
    int32_t *h_tok = h, *h_pos = h + n, *h_seq = h + 2 * n, *h_slot = h + 3 * n, *h_want = h_slot + B;
    memcpy(h_tok, p.tokens.data(), (size_t)n * 4);
    long long max_pos = 0;
    for (size_t i = 0; i < B; i++) {
        for (long long j = 0; j < p.lens[i]; j++) {
            h_pos[row0[i] + j] = (int32_t)(p.pos0[i] + j);
            h_seq[row0[i] + j] = (int32_t)i;
        }
        h_slot[i] = p.slots[i];
        max_pos = std::max(max_pos, p.pos0[i] + p.lens[i] - 1);
    }
    {
        long long r = 0;
        for (size_t i = 0; i < B; i++)
            for (long long w = 0; w < entries[i].n_want; w++) h_want[r++] = (int32_t)(row0[i] + entries[i].want[w]);
    }
    int32_t *h_tab = h_want + p.n_want;
    std::vector<size_t> tab_off;
    for (size_t gi = 0; gi < cache->groups.size(); gi++) {
        tab_off.push_back((size_t)(h_tab - h));
        cache->block_table(*cache->groups[gi], p.slots, widths[gi], h_tab);
        h_tab += B * (size_t)widths[gi];
    }
    Buf in = dev->pool.get(total * 4);
    dev->upload_pinned(in.ptr, h, total * 4);
    const int32_t *d = in.as<int32_t>();

    StepContext ctx;
    ctx.kind = p.kind;
    ctx.dtype = dtype;
    ctx.dev = dev.get();
    ctx.n_rows = n;
    ctx.n_seqs = (int)B;
    ctx.hidden = model->spec.hidden_size;
    ctx.row_pos = d + n;
    ctx.row_seq = d + 2 * n;
    ctx.seq_slot = d + 3 * n;
    ctx.seq_slots = p.slots;
    ctx.seq_pos0 = p.pos0;
    ctx.seq_len = p.lens;
    ctx.seq_row0 = row0;
    ctx.max_pos = max_pos;
    ctx.trace = trace;
    std::map<const KVGroup *, std::pair<const int32_t *, int>> bt;
    for (size_t gi = 0; gi < cache->groups.size(); gi++)
        bt[cache->groups[gi].get()] = {d + tab_off[gi], widths[gi]};
    std::vector<LayerCache> caches = layer_caches(bt);
    Buf logits = model->forward(ctx, d, caches, all_rows ? nullptr : d + 3 * n + B, all_rows ? -1 : p.n_want);
    cache->advance(p.slots, p.lens);
    if (n_wanted) *n_wanted = p.n_want;
    return logits;
}

// ---------------------------------------------------------------- decode
void Engine::drop_graphs() {
    if (graphs_.empty()) return;
    cudaStreamSynchronize(dev->stream);
    graphs_.clear();
    last_graph_ = nullptr;
    last_slots_.clear();
}

SamplerScratch &Engine::sampler_scratch() {
    if (!sampler_scratch_) {
        long long vocab = model->spec.vocab_size, cap = 1;
        while (cap < vocab) cap *= 2;
        dev->make_current();
        sampler_scratch_.reset(new SamplerScratch());
        sampler_scratch_->cap = cap;
        sampler_scratch_->keys = dev->tensor(I64, {cache->max_seqs, cap});
        sampler_scratch_->probs = dev->tensor(F32, {cache->max_seqs, cap});
    }
    return *sampler_scratch_;
}

bool Engine::needs_long_way(float temperature, int top_k) const {
    return temperature > 0 && ops::sample_needs_big((int)model->spec.vocab_size, top_k);
}

std::vector<int32_t> Engine::pick(const float *logits, const std::vector<int> &slots, bool sampled,
                                  bool long_way, int *forced) {
    dev->make_current();
    int rows = (int)slots.size();
    int vocab = (int)model->spec.vocab_size;
    Buf out = dev->pool.get((size_t)rows * 4 * 3);
    int32_t *o = out.as<int32_t>();
    ops::SamplerArrays s;
    if (sampled) {
        cache->ensure_samplers(slots);
        for (int sl1 : slots)
            long_way = long_way || needs_long_way(cache->sampler(sl1).temperature, cache->sampler(sl1).top_k);
        std::vector<int32_t> sl(slots.begin(), slots.end());
        dev->upload(o + rows, sl.data(), (size_t)rows * 4);
        s.row_slot = o + rows;
        s.temperature = (const float *)cache->temperature.ptr;
        s.top_k = (const int32_t *)cache->top_k.ptr;
        s.top_p = (const float *)cache->top_p.ptr;
        s.min_p = (const float *)cache->min_p.ptr;
        s.rng = (unsigned long long *)cache->rng.ptr;
        s.forced = o + 2 * rows;
        if (long_way) {
            SamplerScratch &sc = sampler_scratch();
            s.big_keys = (unsigned long long *)sc.keys.ptr;
            s.big_probs = (float *)sc.probs.ptr;
            s.big_cap = sc.cap;
        }
    }
    ops::sample(*dev, logits, rows, vocab, s, o);
    std::vector<int32_t> host((size_t)rows * 3);
    cuda_check(cudaMemcpyAsync(host.data(), o, (size_t)rows * 4 * (sampled ? 3 : 1), cudaMemcpyDeviceToHost,
                               dev->stream), "reading the chosen tokens");
    dev->sync();
    int f = 0;
    for (int i = 0; i < rows; i++) {
        if (host[(size_t)i] < 0)
            fail(JB_LLM_EFAIL, "the sampler had no scratch for a row that keeps all its candidates");
        if (sampled) f += host[(size_t)(2 * rows + i)];
    }
    if (forced) *forced = f;
    host.resize((size_t)rows);
    return host;
}

PendingDecode *Engine::decode_begin(const std::vector<int> &slots, const int32_t *tokens, bool sampled,
                                    bool long_way) {
    dev->make_current();
    if (sampled) {
        // a slot whose settings were never set draws greedily; the long way is taken
        // when any row's settings ask for it
        for (int s : slots)
            if (!cache->slots.live(s)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", s));
        cache->ensure_samplers(slots);
        for (int s : slots)
            long_way = long_way || needs_long_way(cache->sampler(s).temperature, cache->sampler(s).top_k);
    }
    long_way = long_way && sampled;
    std::vector<int32_t> feed(slots.size(), 0);
    if (!tokens) {
        if (!use_graphs || !last_graph_ || last_slots_ != slots)
            fail(JB_LLM_EINVAL, "a step can go on from the device's own tokens only right after a decode "
                                "step of the same sequences");
    } else {
        feed.assign(tokens, tokens + slots.size());
    }
    std::vector<StepEntry> entries;
    static const int32_t zero = 0;
    for (size_t i = 0; i < slots.size(); i++) entries.push_back(StepEntry{slots[i], &feed[i], 1, &zero, 1});
    if (!use_graphs) {
        long long nw = 0;
        Buf logits = step(entries, &nw);
        eager_pending_ = PendingDecode();
        eager_pending_.tokens = pick(logits.as<float>(), slots, sampled, long_way, nullptr);
        eager_pending_.n = (int)slots.size();
        eager_pending_.taken = true;
        return &eager_pending_;
    }
    Plan p = plan(entries);
    cache->reserve(p.slots, p.lens);
    // launch sizes are fixed for positions below bound: a new graph every 256
    // positions keeps them close to what the step needs
    long long need = *std::max_element(p.pos0.begin(), p.pos0.end()) + 1;
    long long bound = std::min((need + 255) / 256 * 256, max_positions);
    GraphKey key((int)slots.size(), bound, sampled, long_way);
    DecodeGraph *g = nullptr;
    for (auto it = graphs_.begin(); it != graphs_.end(); ++it) {
        if (it->first == key) {
            graphs_.splice(graphs_.end(), graphs_, it);     // used last: to the back
            g = graphs_.back().second.get();
            break;
        }
    }
    if (!g) {
        while (graphs_.size() >= std::max<size_t>(max_graphs, 1)) {
            // a step of the graph that goes may still be under way
            dev->sync();
            if (graphs_.front().second.get() == last_graph_) {
                last_graph_ = nullptr;
                last_slots_.clear();
                if (!tokens) fail(JB_LLM_EFAIL, "the step before this one lost its graph");
            }
            graphs_.pop_front();
        }
        graphs_.emplace_back(key, std::unique_ptr<DecodeGraph>(
                                      new DecodeGraph(*this, (int)slots.size(), bound, sampled, long_way)));
        g = graphs_.back().second.get();
    }
    DecodeGraph *before = tokens ? nullptr : last_graph_;
    PendingDecode *pending = g->begin(slots, tokens ? p.tokens.data() : nullptr, p.pos0, before);
    last_graph_ = g;
    last_slots_ = slots;
    cache->advance(p.slots, p.lens);
    return pending;
}

void Engine::check_device_errors() {
    dev->make_current();
    dev->sync();
    int a = ops::gemm_tc_error(), b = ops::attn_tc_error();
    if (a != 0 || b != 0)
        fail(JB_LLM_EFAIL, fmt("a tensor-core kernel gave up a bounded wait (product: code %d, attention: "
                               "code %d); what was computed since the last check is not valid", a, b));
}

Json Engine::describe() const {
    Json o = Json::object();
    o.set("architecture", model->spec.architecture);
    o.set("dtype", dtype_name(dtype));
    o.set("vocab_size", model->spec.vocab_size);
    o.set("hidden_size", model->spec.hidden_size);
    o.set("max_positions", max_positions);
    o.set("n_layers", (long long)model->spec.layers.size());
    o.set("run_order", (long long)model->spec.run_order.size());
    o.set("weight_bytes", (unsigned long long)model->weight_bytes());
    o.set("use_graphs", use_graphs);
    o.set("graphs", (long long)graphs_.size());
    o.set("graph_captures", graph_captures);
    o.set("device", dev->index);
    o.set("sm_count", dev->sm_count);
    o.set("pool_bytes", (unsigned long long)dev->pool.reserved());
    o.set("pool_allocations", dev->pool.allocations());
    o.set("h2d_bytes", dev->h2d_bytes);
    o.set("launches", ops::launches());
    o.set("cache", cache->describe());
    if (config) {
        o.set("config", config->to_json());
        Json eos = Json::array();
        for (int t : config->eos_token_ids()) eos.push(t);
        o.set("eos_token_ids", eos);
    }
    o.set("spec", model->spec.to_json());
    return o;
}

}  // namespace jb
