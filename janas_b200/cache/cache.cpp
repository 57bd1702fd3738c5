#include "cache.h"

#include <algorithm>
#include <set>

#include "../csrc/kernels.h"

namespace jb {

// ------------------------------------------------------------------- pools
PagePool::PagePool(int n_pages, std::string name) : n_pages_(n_pages), name_(std::move(name)) {
    if (n_pages <= 0) fail(JB_LLM_EINVAL, "a page pool needs at least one page");
    for (int p = n_pages - 1; p >= 0; p--) free_.push_back(p);
    held_.assign((size_t)n_pages, 0);
}

std::vector<int> PagePool::take(int count) {
    if (count > (int)free_.size())
        throw CacheFull(fmt("%s: %d pages wanted, %zu of %d free (%d tokens in all)", name_.c_str(),
                            count, free_.size(), n_pages_, n_pages_ * PAGE));
    std::vector<int> got;
    for (int i = 0; i < count; i++) {
        got.push_back(free_.back());
        free_.pop_back();
        held_[(size_t)got.back()] = 1;
    }
    return got;
}

void PagePool::give_back(const std::vector<int> &pages) {
    for (int p : pages) {
        if (p < 0 || p >= n_pages_ || !held_[(size_t)p])
            fail(JB_LLM_EFAIL, fmt("%s: page %d given back but not held", name_.c_str(), p));
        held_[(size_t)p] = 0;
        free_.push_back(p);
    }
}

void PagePool::check() const {
    std::set<int> fr(free_.begin(), free_.end());
    if (fr.size() != free_.size()) fail(JB_LLM_EFAIL, name_ + ": a page is free twice");
    for (int p = 0; p < n_pages_; p++) {
        bool held = held_[(size_t)p] != 0;
        if (held == (fr.count(p) > 0))
            fail(JB_LLM_EFAIL, fmt("%s: page %d is %s", name_.c_str(), p, held ? "held and free" : "lost"));
    }
}

SlotPool::SlotPool(int n_slots) : n_slots_(n_slots) {
    if (n_slots <= 0) fail(JB_LLM_EINVAL, "at least one slot is needed");
    for (int s = n_slots - 1; s >= 0; s--) free_.push_back(s);
    live_.assign((size_t)n_slots, 0);
}

int SlotPool::take() {
    if (free_.empty()) throw CacheFull(fmt("all %d sequence slots are in use", n_slots_));
    int s = free_.back();
    free_.pop_back();
    live_[(size_t)s] = 1;
    return s;
}

void SlotPool::give_back(int slot) {
    if (!live(slot)) fail(JB_LLM_EFAIL, fmt("slot %d given back but not in use", slot));
    live_[(size_t)slot] = 0;
    free_.push_back(slot);
}

void SlotPool::check() const {
    std::set<int> fr(free_.begin(), free_.end());
    if (fr.size() != free_.size()) fail(JB_LLM_EFAIL, "a slot is free twice");
    for (int s = 0; s < n_slots_; s++) {
        bool lv = live_[(size_t)s] != 0;
        if (lv == (fr.count(s) > 0))
            fail(JB_LLM_EFAIL, fmt("slot %d is %s", s, lv ? "live and free" : "lost"));
    }
}

// ------------------------------------------------------------------ groups
KVGroup::KVGroup(KVSpec sp, std::vector<int> ents, int n_pages, int n_slots)
    : spec(sp), entries(std::move(ents)),
      pool(n_pages, fmt("cache group (kv_heads %d, head_dim %d, window %d)", sp.num_kv_heads,
                        sp.head_dim, sp.window)) {
    for (size_t i = 0; i < entries.size(); i++) index[entries[i]] = (int)i;
    pages.resize((size_t)n_slots);
}

size_t KVGroup::entry_bytes() const {
    return (size_t)pool.n_pages() * (size_t)spec.num_kv_heads * PAGE * (size_t)spec.head_dim *
           dtype_size(k.dt);
}

int KVGroup::first_needed_page(long long next_pos) const {
    if (!spec.window) return 0;
    return (int)(std::max(0ll, next_pos + 1 - spec.window) / PAGE);
}

void KVGroup::extend(int slot, long long end) {
    auto &have = pages[(size_t)slot];
    long long want = pages_for(end);
    if (want > (long long)have.size()) {
        auto got = pool.take((int)(want - (long long)have.size()));
        have.insert(have.end(), got.begin(), got.end());
    }
}

void KVGroup::release_unseen(int slot, long long next_pos) {
    auto &have = pages[(size_t)slot];
    int first = std::min(first_needed_page(next_pos), (int)have.size());
    std::vector<int> gone;
    for (int i = 0; i < first; i++)
        if (have[(size_t)i] >= 0) { gone.push_back(have[(size_t)i]); have[(size_t)i] = -1; }
    if (!gone.empty()) pool.give_back(gone);
}

void KVGroup::free_slot(int slot) {
    std::vector<int> gone;
    for (int p : pages[(size_t)slot]) if (p >= 0) gone.push_back(p);
    pool.give_back(gone);
    pages[(size_t)slot].clear();
}

int KVGroup::held(int slot) const {
    int n = 0;
    for (int p : pages[(size_t)slot]) n += p >= 0;
    return n;
}

// ------------------------------------------------------------------- cache
Cache::Cache(const std::vector<KVSpec> &kv_specs, const std::vector<StateSpec> &state_specs,
             long long max_tok, int max_sq, DType dt, Device *device)
    : dev(device), dtype(dt), max_tokens(pages_for(max_tok) * PAGE), max_seqs(max_sq),
      slots(max_sq > 0 ? max_sq : 1) {
    if (max_tok <= 0 || max_sq <= 0) fail(JB_LLM_EINVAL, "max_tokens and max_seqs must be positive");
    if (pages_for(max_tok) > (1ll << 30)) fail(JB_LLM_EINVAL, "max_tokens is too large");
    int n_pages = (int)pages_for(max_tok);
    length_.assign((size_t)max_sq, 0);
    sampler_of_.assign((size_t)max_sq, SamplerSettings());
    sampler_set_.assign((size_t)max_sq, 0);
    // groups in the order in which their first entry appears
    std::vector<std::pair<KVSpec, std::vector<int>>> by_spec;
    for (size_t e = 0; e < kv_specs.size(); e++) {
        if (kv_specs[e].none()) continue;
        auto it = std::find_if(by_spec.begin(), by_spec.end(),
                               [&](const std::pair<KVSpec, std::vector<int>> &g) { return g.first == kv_specs[e]; });
        if (it == by_spec.end()) by_spec.push_back({kv_specs[e], {(int)e}});
        else it->second.push_back((int)e);
    }
    for (auto &g : by_spec) {
        groups.emplace_back(new KVGroup(g.first, g.second, n_pages, max_sq));
        KVGroup *grp = groups.back().get();
        grp->k.dt = grp->v.dt = dt;
        std::vector<long long> shape = {(long long)g.second.size(), n_pages, g.first.num_kv_heads, PAGE,
                                        g.first.head_dim};
        if (dev) {
            dev->make_current();
            grp->k = dev->tensor(dt, shape, true);
            grp->v = dev->tensor(dt, shape, true);
        } else {
            grp->k.shape = grp->v.shape = shape;
        }
        for (int e : g.second) group_of[e] = grp;
    }
    for (size_t e = 0; e < state_specs.size(); e++)
        if (!state_specs[e].none()) state_spec[(int)e] = state_specs[e];
    if (dev) {
        rng = dev->tensor(I64, {max_sq}, true);
        temperature = dev->tensor(F32, {max_sq}, true);
        top_k = dev->tensor(I32, {max_sq}, true);
        top_p = dev->tensor(F32, {max_sq}, true);
        min_p = dev->tensor(F32, {max_sq}, true);
        for (auto &kv : state_spec) {
            std::vector<long long> shape = {max_sq};
            shape.insert(shape.end(), kv.second.shape.begin(), kv.second.shape.end());
            mixer_state[kv.first] = dev->tensor(kv.second.dtype, shape, true);
        }
    }
}

void Cache::zero_state(int slot) {
    if (!dev) return;
    for (auto &kv : mixer_state) {
        size_t b = state_spec[kv.first].bytes();
        cuda_check(cudaMemsetAsync((char *)kv.second.ptr + (size_t)slot * b, 0, b, dev->stream),
                   "clearing a sequence's state");
    }
}

int Cache::new_sequence() {
    int slot = slots.take();
    length_[(size_t)slot] = 0;
    sampler_of_[(size_t)slot] = SamplerSettings();
    sampler_set_[(size_t)slot] = 0;
    try {
        zero_state(slot);
    } catch (...) {
        slots.give_back(slot);
        throw;
    }
    return slot;
}

void Cache::free_sequence(int slot) {
    if (!slots.live(slot)) fail(JB_LLM_EINVAL, fmt("slot %d freed but not in use", slot));
    for (auto &g : groups) g->free_slot(slot);
    slots.give_back(slot);
    length_[(size_t)slot] = 0;
}

bool Cache::can_truncate(int slot, long long n) const {
    if (!slots.live(slot) || n < 0 || n > length_[(size_t)slot]) return false;
    if (n == 0 || n == length_[(size_t)slot]) return true;
    if (!state_spec.empty()) return false;
    for (auto &g : groups) {
        auto &have = g->pages[(size_t)slot];
        for (long long i = g->first_needed_page(n); i < pages_for(n); i++)
            if (have[(size_t)i] < 0) return false;
    }
    return true;
}

bool Cache::truncate(int slot, long long n) {
    if (!can_truncate(slot, n)) return false;
    if (n == length_[(size_t)slot]) return true;
    for (auto &g : groups) {
        auto &have = g->pages[(size_t)slot];
        size_t keep = (size_t)pages_for(n);
        std::vector<int> gone;
        for (size_t i = keep; i < have.size(); i++) if (have[i] >= 0) gone.push_back(have[i]);
        if (!gone.empty()) g->pool.give_back(gone);
        if (have.size() > keep) have.resize(keep);
    }
    length_[(size_t)slot] = n;
    if (n == 0) zero_state(slot);
    return true;
}

void Cache::set_samplers(const std::vector<int> &sl, const std::vector<SamplerSettings> &s) {
    if (sl.size() != s.size()) fail(JB_LLM_EINVAL, "set_samplers: one setting per slot");
    for (int slot : sl)
        if (!slots.live(slot)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", slot));
    for (size_t i = 0; i < sl.size(); i++) {
        sampler_of_[(size_t)sl[i]] = s[i];
        sampler_set_[(size_t)sl[i]] = 1;
    }
    if (!dev || sl.empty()) return;
    // packed on the host as [slots | seeds | temperature | top_k | top_p | min_p], one
    // copy, then a kernel writes each value to its slot's place
    size_t n = sl.size();
    size_t bytes = n * (4 + 8 + 4 + 4 + 4 + 4) + 8;
    char *h = (char *)dev->pinned(bytes);
    unsigned long long *seeds = (unsigned long long *)h;
    int32_t *sl_h = (int32_t *)(h + 8 * n);
    float *temp = (float *)(h + 12 * n);
    int32_t *tk = (int32_t *)(h + 16 * n);
    float *tp = (float *)(h + 20 * n), *mp = (float *)(h + 24 * n);
    for (size_t i = 0; i < n; i++) {
        seeds[i] = s[i].seed;
        sl_h[i] = sl[i];
        temp[i] = s[i].temperature;
        tk[i] = s[i].top_k;
        tp[i] = s[i].top_p;
        mp[i] = s[i].min_p;
    }
    Buf d = dev->pool.get(bytes);
    dev->upload_pinned(d.ptr, h, bytes);
    char *p = (char *)d.ptr;
    int rc = jb_sampler_set((const int32_t *)(p + 8 * n), (int)n, (const unsigned long long *)p,
                            (const float *)(p + 12 * n), (const int32_t *)(p + 16 * n),
                            (const float *)(p + 20 * n), (const float *)(p + 24 * n),
                            (unsigned long long *)rng.ptr, (float *)temperature.ptr,
                            (int32_t *)top_k.ptr, (float *)top_p.ptr, (float *)min_p.ptr, dev->stream);
    if (rc != 0) fail(JB_LLM_EFAIL, "the sampler settings could not be written");
}

void Cache::ensure_samplers(const std::vector<int> &sl) {
    std::vector<int> unset;
    for (int slot : sl)
        if (slots.live(slot) && !sampler_set_[(size_t)slot]) unset.push_back(slot);
    if (!unset.empty()) set_samplers(unset, std::vector<SamplerSettings>(unset.size()));
}

void Cache::reserve(const std::vector<int> &sl, const std::vector<long long> &counts) {
    struct Taken { KVGroup *g; int slot; size_t before; };
    std::vector<Taken> taken;
    try {
        for (size_t i = 0; i < sl.size(); i++) {
            int slot = sl[i];
            if (!slots.live(slot)) fail(JB_LLM_EINVAL, fmt("slot %d is not in use", slot));
            long long end = length_[(size_t)slot] + counts[i];
            for (auto &g : groups) {
                taken.push_back({g.get(), slot, g->pages[(size_t)slot].size()});
                g->extend(slot, end);
            }
        }
    } catch (...) {
        for (auto &t : taken) {
            auto &have = t.g->pages[(size_t)t.slot];
            if (have.size() > t.before) {
                std::vector<int> extra(have.begin() + (long)t.before, have.end());
                t.g->pool.give_back(extra);
                have.resize(t.before);
            }
        }
        throw;
    }
}

void Cache::advance(const std::vector<int> &sl, const std::vector<long long> &counts) {
    for (size_t i = 0; i < sl.size(); i++) {
        length_[(size_t)sl[i]] += counts[i];
        long long nxt = length_[(size_t)sl[i]];
        for (auto &g : groups)
            if (g->spec.window) g->release_unseen(sl[i], nxt);
    }
}

int Cache::table_width(const KVGroup &g, const std::vector<int> &sl) const {
    size_t w = 1;
    for (int s : sl) w = std::max(w, g.pages[(size_t)s].size());
    return (int)((w + 7) / 8 * 8);
}

void Cache::block_table(const KVGroup &g, const std::vector<int> &sl, int width, int32_t *out) const {
    for (size_t i = 0; i < sl.size(); i++) {
        auto &pg = g.pages[(size_t)sl[i]];
        int32_t *row = out + i * (size_t)width;
        size_t n = std::min(pg.size(), (size_t)width);
        for (size_t j = 0; j < n; j++) row[j] = pg[j];
        for (size_t j = n; j < (size_t)width; j++) row[j] = -1;
    }
}

long long Cache::tokens_held() const {
    long long m = 0;
    for (auto &g : groups) m = std::max(m, (long long)(g->pool.n_pages() - g->pool.n_free()) * PAGE);
    return m;
}

size_t Cache::bytes() const {
    size_t b = 0;
    for (auto &g : groups) {
        size_t n = dtype_size(dtype);
        for (auto s : g->k.shape) n *= (size_t)s;
        b += 2 * n;
    }
    return b;
}

void Cache::check() const {
    slots.check();
    for (auto &g : groups) {
        g->pool.check();
        std::set<int> seen;
        for (size_t slot = 0; slot < g->pages.size(); slot++) {
            auto &pages = g->pages[slot];
            if (!pages.empty() && !slots.live((int)slot))
                fail(JB_LLM_EFAIL, fmt("free slot %zu still holds pages", slot));
            for (int p : pages) {
                if (p < 0) continue;
                if (!seen.insert(p).second) fail(JB_LLM_EFAIL, fmt("page %d is held twice", p));
            }
        }
        if ((int)seen.size() != g->pool.n_pages() - g->pool.n_free())
            fail(JB_LLM_EFAIL, "pages held by nobody");
    }
}

Json Cache::describe() const {
    Json o = Json::object();
    o.set("max_tokens", max_tokens);
    o.set("max_seqs", max_seqs);
    o.set("dtype", dtype_name(dtype));
    o.set("page", PAGE);
    o.set("bytes", (unsigned long long)bytes());
    o.set("free_slots", slots.n_free());
    Json gs = Json::array();
    for (auto &g : groups) {
        Json j = Json::object();
        j.set("num_kv_heads", g->spec.num_kv_heads);
        j.set("head_dim", g->spec.head_dim);
        j.set("window", g->spec.window);
        Json es = Json::array();
        for (int e : g->entries) es.push(e);
        j.set("entries", es);
        Json sh = Json::array();
        for (auto s : g->k.shape) sh.push(s);
        j.set("shape", sh);
        j.set("n_pages", g->pool.n_pages());
        j.set("free_pages", g->pool.n_free());
        j.set("k", (unsigned long long)(uintptr_t)g->k.ptr);
        j.set("v", (unsigned long long)(uintptr_t)g->v.ptr);
        gs.push(j);
    }
    o.set("groups", gs);
    Json st = Json::array();
    for (auto &kv : state_spec) st.push(kv.first);
    o.set("state_entries", st);
    return o;
}

}  // namespace jb
