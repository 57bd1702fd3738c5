#include "generate.h"

#include <algorithm>
#include <chrono>
#include <map>

namespace jb {

static double now() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

const char *finish_name(int f) {
    switch (f) {
        case FINISH_STOP: return "stop";
        case FINISH_LENGTH: return "length";
        case FINISH_CONTEXT: return "context";
    }
    return "";
}

void GenOptions::validate() const {
    if ((int)stop.size() > MAX_STOP) fail(JB_LLM_EINVAL, fmt("at most %d stop tokens besides eos", MAX_STOP));
    if (!(temperature >= 0) || !(top_p >= 0 && top_p <= 1) || !(min_p >= 0 && min_p <= 1) || top_k < 0)
        fail(JB_LLM_EINVAL, "temperature >= 0, top_k >= 0, top_p and min_p within [0, 1]");
}

bool GenOptions::is_stop(int token) const {
    if (eos >= 0 && token == eos) return true;
    return std::find(stop.begin(), stop.end(), token) != stop.end();
}

// ------------------------------------------------------------------ decisions
long long tokens_needed(long long prompt_len, long long max_new, long long max_positions) {
    return pages_for(std::min(prompt_len + std::max(max_new - 1, 0ll), max_positions)) * PAGE;
}

std::vector<std::vector<int>> plan_batches(const std::vector<long long> &prompt_lens,
                                           const std::vector<long long> &max_news, int max_batch,
                                           long long max_tokens, long long max_positions) {
    if (max_batch <= 0) throw CacheFull("no sequence slot is free");
    std::vector<std::vector<int>> batches;
    std::vector<int> cur;
    long long used = 0;
    for (size_t i = 0; i < prompt_lens.size(); i++) {
        long long need = tokens_needed(prompt_lens[i], max_news[i], max_positions);
        if (need > max_tokens)
            throw CacheFull(fmt("request %zu: %lld prompt tokens and %lld new ones need %lld tokens of "
                                "cache, the cache has %lld free", i, prompt_lens[i], max_news[i], need,
                                max_tokens));
        if (!cur.empty() && ((int)cur.size() >= max_batch || used + need > max_tokens)) {
            batches.push_back(cur);
            cur.clear();
            used = 0;
        }
        cur.push_back((int)i);
        used += need;
    }
    if (!cur.empty()) batches.push_back(cur);
    return batches;
}

int finish_reason(int token, long long n_generated, long long max_new, long long length,
                  long long max_positions, const GenOptions &o) {
    if (o.is_stop(token)) return FINISH_STOP;
    if (n_generated >= max_new) return FINISH_LENGTH;
    if (length + 1 > max_positions) return FINISH_CONTEXT;
    return FINISH_NONE;
}

bool goes_on_unless_stopped(long long n_generated, long long max_new, long long length,
                            long long max_positions) {
    return n_generated < max_new && length + 1 <= max_positions;
}

// ----------------------------------------------------------------------- loop
std::vector<Result> generate(Driver &d, const std::vector<Request> &requests, int max_batch, GenStats *stats) {
    for (size_t i = 0; i < requests.size(); i++) {
        const Request &r = requests[i];
        r.options.validate();
        if (r.prompt.empty()) fail(JB_LLM_EINVAL, fmt("request %zu: the prompt is empty", i));
        if ((long long)r.prompt.size() > d.max_positions())
            fail(JB_LLM_ELIMIT, fmt("request %zu: the prompt has %zu tokens, the context %lld", i,
                                    r.prompt.size(), d.max_positions()));
        for (int32_t t : r.prompt)
            if (t < 0 || t >= d.vocab_size())
                fail(JB_LLM_EINVAL, fmt("request %zu: a token id lies outside the vocabulary of %lld", i,
                                        d.vocab_size()));
    }
    GenStats local;
    GenStats &st = stats ? *stats : local;
    std::vector<Result> results(requests.size());
    std::vector<long long> plens, news;
    for (auto &r : requests) {
        plens.push_back((long long)r.prompt.size());
        news.push_back(r.max_new);
    }
    // batches are planned against what is free now: open sessions and slots taken by
    // the caller hold slots and pages that this call cannot use
    auto plan = plan_batches(plens, news, std::min(max_batch, d.free_slots()), d.free_tokens(),
                             d.max_positions());
    for (auto &batch : plan) {
        st.batches++;
        std::vector<int> live;
        for (int i : batch) {
            if (requests[(size_t)i].max_new > 0) live.push_back(i);
            else results[(size_t)i].finish = FINISH_LENGTH;
        }
        if (live.empty()) continue;
        std::map<int, int> slots;       // request -> slot, while it is going
        try {
            for (int i : live) slots[i] = d.new_sequence();
            bool sampled = false, long_way = false;
            for (int i : live) {
                const GenOptions &o = requests[(size_t)i].options;
                sampled = sampled || o.temperature > 0;
                long_way = long_way || d.needs_long_way(o.temperature, o.top_k);
            }
            if (sampled) {
                std::vector<int> sl;
                std::vector<SamplerSettings> ss;
                for (int i : live) {
                    sl.push_back(slots[i]);
                    ss.push_back(requests[(size_t)i].options.sampler());
                }
                d.set_samplers(sl, ss);
            }
            std::map<int, std::vector<int32_t>> out;
            double t0 = now();
            std::vector<FeedEntry> entries;
            for (int i : live) {
                const Request &r = requests[(size_t)i];
                st.prompt_tokens += (uint32_t)r.prompt.size();
                entries.push_back(FeedEntry{slots[i], r.prompt.data(), (long long)r.prompt.size(), true});
            }
            int forced = 0;
            std::vector<int32_t> toks = d.run(entries, sampled, long_way, &forced);
            st.prefill_seconds += now() - t0;
            std::vector<int> active = live;
            // Decode steps are launched one ahead where the engine can feed a step the
            // tokens of the step before it on the device: while step t runs, step
            // t + 1 is already queued behind it, and the host reads t's tokens
            // meanwhile.  That is done only when every sequence is sure to go on
            // unless it draws a stop token; one that does has run one step too many,
            // which changes nothing for the others, and the loop then takes the
            // remaining sequences' tokens from that step before it goes on.
            bool ahead_ok = d.decodes_ahead();
            void *ahead = nullptr;          // the step under way beyond toks, and its rows
            std::vector<int> ahead_rows;
            while (true) {
                st.forced_tokens += (uint32_t)forced;
                forced = 0;
                std::vector<int> nxt;
                std::vector<int32_t> feed;
                for (size_t k = 0; k < active.size(); k++) {
                    int i = active[k];
                    int32_t tok = toks[k];
                    const Request &r = requests[(size_t)i];
                    out[i].push_back(tok);
                    st.new_tokens++;
                    long long held = d.length(slots[i]) - (ahead ? 1 : 0);
                    int why = finish_reason(tok, (long long)out[i].size(), r.max_new, held, d.max_positions(),
                                            r.options);
                    if (why == FINISH_NONE) {
                        nxt.push_back(i);
                        feed.push_back(tok);
                    } else {
                        results[(size_t)i].tokens = out[i];
                        results[(size_t)i].finish = why;
                        int s = slots[i];
                        slots.erase(i);
                        d.free_sequence(s);
                    }
                }
                bool ended = nxt.size() != active.size();
                active = nxt;
                t0 = now();
                if (ahead && (ended || active.empty())) {
                    // the step under way ran with sequences that have ended: the
                    // others' tokens are good
                    std::vector<int32_t> got = d.decode_end(ahead);
                    st.passes++;
                    st.d2h_bytes += 4 * ahead_rows.size();
                    st.decode_seconds += now() - t0;
                    toks.clear();
                    for (int i : active) {
                        size_t at = (size_t)(std::find(ahead_rows.begin(), ahead_rows.end(), i) - ahead_rows.begin());
                        toks.push_back(got.at(at));
                    }
                    ahead = nullptr;
                    if (active.empty()) break;
                    continue;
                }
                if (active.empty()) break;
                unsigned long long h2d0 = d.h2d_bytes();
                std::vector<int> cur_slots;
                for (int i : active) cur_slots.push_back(slots[i]);
                void *cur = nullptr;
                if (ahead) {
                    cur = ahead;
                    ahead = nullptr;
                } else if (ahead_ok) {
                    cur = d.decode_begin(cur_slots, feed.data(), sampled, long_way);
                } else {
                    std::vector<FeedEntry> es;
                    for (size_t k = 0; k < active.size(); k++)
                        es.push_back(FeedEntry{cur_slots[k], &feed[k], 1, true});
                    toks = d.run(es, sampled, long_way, &forced);
                }
                if (cur) {
                    bool all_go_on = true;
                    for (int i : active)
                        all_go_on = all_go_on &&
                                    goes_on_unless_stopped((long long)out[i].size() + 1, requests[(size_t)i].max_new,
                                                           d.length(slots[i]), d.max_positions());
                    if (all_go_on) {
                        ahead = d.decode_begin(cur_slots, nullptr, sampled, long_way);
                        ahead_rows = active;
                    }
                    toks = d.decode_end(cur);
                }
                st.passes++;
                st.decode_seconds += now() - t0;
                st.h2d_bytes += d.h2d_bytes() - h2d0;
                st.d2h_bytes += 4 * active.size();
            }
        } catch (...) {
            for (auto &kv : slots) {
                try { d.free_sequence(kv.second); } catch (...) {}
            }
            throw;
        }
        for (auto &kv : slots) d.free_sequence(kv.second);
    }
    d.check_errors();
    return results;
}

// ------------------------------------------------------------------ sessions
Session::Session(Driver &d, const GenOptions &o) : driver(d) {
    slot = d.new_sequence();
    try {
        set_options(o);
    } catch (...) {
        close();
        throw;
    }
}

Session::~Session() {
    try { close(); } catch (...) {}
}

static int slot_of(const Session &s) {
    if (s.slot < 0) fail(JB_LLM_EINVAL, "the session is closed");
    return s.slot;
}

long long Session::computed() const { return driver.length(slot_of(*this)); }

void Session::set_options(const GenOptions &o) {
    o.validate();
    int s = slot_of(*this);
    options = o;
    driver.set_samplers({s}, {o.sampler()});
}

void Session::append(const int32_t *tokens, long long n) {
    slot_of(*this);
    for (long long i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= driver.vocab_size())
            fail(JB_LLM_EINVAL, fmt("a token id lies outside the vocabulary of %lld", driver.vocab_size()));
    if ((long long)hist.size() + n > driver.max_positions() + 1)
        fail(JB_LLM_EFULL, fmt("%zu + %lld tokens do not fit the context of %lld", hist.size(), n,
                               driver.max_positions()));
    hist.insert(hist.end(), tokens, tokens + n);
}

void Session::truncate(long long n) {
    if (n < 0 || n > (long long)hist.size())
        fail(JB_LLM_EINVAL, fmt("cannot keep %lld of %zu tokens", n, hist.size()));
    int s = slot_of(*this);
    hist.resize((size_t)n);
    // of the kept tokens the last one is computed again by the next pass (its logits
    // are needed); where the cache cannot go back, all of them are
    long long keep = std::min(computed(), std::max(n - 1, 0ll));
    if (!driver.truncate_sequence(s, keep)) driver.truncate_sequence(s, 0);
}

void Session::close() {
    if (slot >= 0) {
        int s = slot;
        slot = -1;
        driver.free_sequence(s);
    }
}

namespace {
struct Item { Session *s; long long count; bool want; };

// Runs, for each item, the next `count` tokens that the session has not computed;
// returns the chosen token of every item that wants one, in the items' order.  One
// pass where the model can take it: all sequences at their start, all with one
// token, or (models whose mixers can append several tokens to a sequence that
// holds some) any mixture.  Else the sequences at their start go first, and the
// others go on token by token together.
std::vector<int32_t> feed(Driver &d, const std::vector<Item> &items, bool sampled, bool long_way, int *forced) {
    auto entries_of = [](const std::vector<Item> &part, const std::vector<long long> &counts,
                         const std::vector<char> &wants) {
        std::vector<FeedEntry> es;
        for (size_t i = 0; i < part.size(); i++) {
            Session *s = part[i].s;
            es.push_back(FeedEntry{s->slot, s->hist.data() + s->computed(), counts[i], wants[i] != 0});
        }
        return es;
    };
    std::vector<Item> starts, others;
    for (auto &it : items) (it.s->computed() == 0 ? starts : others).push_back(it);
    bool one_step = others.empty() || starts.empty();
    for (auto &it : others) one_step = one_step && it.count == 1;
    if (forced) *forced = 0;
    if (one_step || d.supports_extend()) {
        std::vector<long long> counts;
        std::vector<char> wants;
        for (auto &it : items) { counts.push_back(it.count); wants.push_back(it.want); }
        return d.run(entries_of(items, counts, wants), sampled, long_way, forced);
    }
    std::map<Session *, int32_t> got;
    int f = 0, f1 = 0;
    if (!starts.empty()) {
        std::vector<long long> counts;
        std::vector<char> wants;
        for (auto &it : starts) { counts.push_back(it.count); wants.push_back(it.want); }
        std::vector<int32_t> t = d.run(entries_of(starts, counts, wants), sampled, long_way, &f1);
        f += f1;
        size_t k = 0;
        for (auto &it : starts) if (it.want) got[it.s] = t.at(k++);
    }
    std::map<Session *, long long> left;
    for (auto &it : others) left[it.s] = it.count;
    while (true) {
        std::vector<Item> part;
        for (auto &it : others) if (left[it.s] > 0) part.push_back(it);
        if (part.empty()) break;
        std::vector<long long> counts(part.size(), 1);
        std::vector<char> wants;
        for (auto &it : part) wants.push_back(it.want && left[it.s] == 1);
        std::vector<int32_t> t = d.run(entries_of(part, counts, wants), sampled, long_way, &f1);
        f += f1;
        size_t k = 0;
        for (size_t i = 0; i < part.size(); i++) {
            left[part[i].s]--;
            if (wants[i]) got[part[i].s] = t.at(k++);
        }
    }
    if (forced) *forced = f;
    std::vector<int32_t> out;
    for (auto &it : items) if (it.want) out.push_back(got.at(it.s));
    return out;
}
}  // namespace

void Session::prefill() {
    long long n = (long long)hist.size() - 1 - computed();
    if (n > 0) {
        double t0 = now();
        feed(driver, {Item{this, n, false}}, false, false, nullptr);
        stats.prompt_tokens += (uint32_t)n;
        stats.prefill_seconds += now() - t0;
    }
}

int Session::next(int32_t *token) {
    int status = 0;
    sessions_step(driver, {this}, token, &status);
    return status;
}

void sessions_step(Driver &d, const std::vector<Session *> &sessions, int32_t *tokens, int *status) {
    std::set<Session *> seen;
    for (Session *s : sessions) {
        if (!s) fail(JB_LLM_EINVAL, "a null session");
        if (!seen.insert(s).second) fail(JB_LLM_EINVAL, "a session appears twice");
        if (&s->driver != &d) fail(JB_LLM_EINVAL, "a session of another engine");
        slot_of(*s);
        if (s->hist.empty()) fail(JB_LLM_EINVAL, "the sequence is empty");
    }
    std::vector<size_t> live;
    for (size_t i = 0; i < sessions.size(); i++) {
        tokens[i] = -1;
        if ((long long)sessions[i]->hist.size() > d.max_positions()) status[i] = 1;
        else { status[i] = 0; live.push_back(i); }
    }
    if (live.empty()) return;
    double t0 = now();
    bool sampled = false, long_way = false;
    std::vector<Item> items;
    bool all_decode = true;
    for (size_t i : live) {
        Session *s = sessions[i];
        sampled = sampled || s->options.temperature > 0;
        long_way = long_way || d.needs_long_way(s->options.temperature, s->options.top_k);
        long long c = (long long)s->hist.size() - s->computed();
        items.push_back(Item{s, c, true});
        all_decode = all_decode && c == 1 && s->computed() > 0;
    }
    std::vector<int32_t> got;
    int forced = 0;
    if (all_decode && d.decodes_ahead()) {
        std::vector<int> slots;
        std::vector<int32_t> last;
        for (auto &it : items) { slots.push_back(it.s->slot); last.push_back(it.s->hist.back()); }
        got = d.decode_end(d.decode_begin(slots, last.data(), sampled, long_way));
    } else {
        got = feed(d, items, sampled, long_way, &forced);
    }
    double dt = now() - t0;
    for (size_t k = 0; k < live.size(); k++) {
        Session *s = items[k].s;
        tokens[live[k]] = got.at(k);
        s->hist.push_back(got[k]);
        s->stats.new_tokens++;
        s->stats.passes++;
        if (live.size() == 1) s->stats.forced_tokens += (uint32_t)forced;
        if (items[k].count > 1) {
            s->stats.prompt_tokens += (uint32_t)(items[k].count - 1);
            s->stats.prefill_seconds += dt;
        } else {
            s->stats.decode_seconds += dt;
        }
    }
    d.check_errors();
}

}  // namespace jb
