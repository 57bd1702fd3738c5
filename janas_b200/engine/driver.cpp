// The engine behind the Driver interface that the generation loop and the
// sessions are written against.
#include "engine.h"
#include "generate.h"

namespace jb {

namespace {

class EngineDriver : public Driver {
public:
    explicit EngineDriver(Engine &e) : e_(e) {}
    long long vocab_size() const override { return e_.model->spec.vocab_size; }
    long long max_positions() const override { return e_.max_positions; }
    int free_slots() const override { return e_.cache->slots.n_free(); }
    long long free_tokens() const override {
        long long t = e_.cache->max_tokens;
        for (auto &g : e_.cache->groups) t = std::min(t, (long long)g->pool.n_free() * PAGE);
        return t;
    }
    int new_sequence() override { return e_.new_sequence(); }
    void free_sequence(int slot) override { e_.free_sequence(slot); }
    long long length(int slot) const override { return e_.length(slot); }
    bool truncate_sequence(int slot, long long n) override { return e_.truncate_sequence(slot, n); }
    void set_samplers(const std::vector<int> &slots, const std::vector<SamplerSettings> &s) override {
        e_.dev->make_current();
        e_.cache->set_samplers(slots, s);
    }
    bool needs_long_way(float temperature, int top_k) const override {
        return e_.needs_long_way(temperature, top_k);
    }
    bool supports_extend() const override { return e_.model->supports(EXTEND); }

    std::vector<int32_t> run(const std::vector<FeedEntry> &entries, bool sampled, bool long_way,
                             int *forced) override {
        std::vector<StepEntry> es;
        std::vector<int32_t> last(entries.size());
        std::vector<int> want_slots;
        for (size_t i = 0; i < entries.size(); i++) {
            last[i] = (int32_t)(entries[i].n - 1);
            es.push_back(StepEntry{entries[i].slot, entries[i].tokens, entries[i].n, &last[i],
                                   entries[i].want ? 1 : 0});
            if (entries[i].want) want_slots.push_back(entries[i].slot);
        }
        long long nw = 0;
        Buf logits = e_.step(es, &nw);
        if (forced) *forced = 0;
        if (want_slots.empty()) return {};
        return e_.pick(logits.as<float>(), want_slots, sampled, long_way && sampled, forced);
    }

    bool decodes_ahead() const override { return e_.decodes_ahead(); }
    void *decode_begin(const std::vector<int> &slots, const int32_t *tokens, bool sampled,
                       bool long_way) override {
        return e_.decode_begin(slots, tokens, sampled, long_way);
    }
    std::vector<int32_t> decode_end(void *pending) override {
        return e_.decode_end((PendingDecode *)pending);
    }
    unsigned long long h2d_bytes() const override { return (unsigned long long)e_.dev->h2d_bytes; }
    void check_errors() override { e_.check_device_errors(); }

private:
    Engine &e_;
};

}  // namespace

std::unique_ptr<Driver> engine_driver(Engine &e) { return std::unique_ptr<Driver>(new EngineDriver(e)); }

}  // namespace jb
