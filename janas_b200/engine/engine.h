// The engine: a model, its cache, and the one step function.
//
// Engine::step runs a batch of sequences that either all start at their first
// token (whole prompts of unequal lengths) or all go on by one token (or, where
// every mixer allows it, any mixture).  It runs only the tokens it is given, as
// one batch of rows, against what earlier steps left in the cache, and returns
// the logits at the wanted places.  There is no padding: the rows are the
// sequences' tokens one after the other, and every kernel finds a row's sequence
// and position in small index arrays.
//
// The reference's batched pass has the same contract: pieces {sequence, tokens,
// n, pos0} run as one block of rows, every weight read once, each piece attending
// over its own sequence's cache, and "each piece's logits are those a pass over
// its tokens alone gives" (src/llm/model.h:193-228, src/llm/model.c:878-912).
// Arguments are checked before any state is touched (src/llm/model.c:651-655,
// 675-678).
//
// Decode steps (one token per sequence, the next token chosen on the device) are
// captured once per (batch size, 256-position bound, sampled or not) into a CUDA
// graph and replayed.  All that changes between steps (positions, slots, block
// tables; the tokens too when the host supplies them) is copied from a pinned
// buffer before the graph runs, and the sampler writes its tokens where the next
// step's embedding reads them, so a step that goes on from them can be queued
// while the step before it still runs.
#pragma once

#include <list>
#include <map>
#include <memory>
#include <tuple>
#include <vector>

#include "../config/registry.h"
#include "model.h"

namespace jb {

// One sequence's share of a step: its next tokens and the places among them
// (indices into tokens) whose logits are wanted.  Host memory.
struct StepEntry {
    int slot = 0;
    const int32_t *tokens = nullptr;
    long long n = 0;
    const int32_t *want = nullptr;
    long long n_want = 0;
};

class Engine;
class DecodeGraph;

// A decode step under way: decode_end waits for it and gives its tokens.
struct PendingDecode {
    cudaEvent_t event = nullptr;        // null: the tokens are there already
    int n = 0;
    const int32_t *out_host = nullptr;  // pinned; valid once the event has passed
    std::vector<int32_t> tokens;        // the result, once taken
    bool taken = false;
    const std::vector<int32_t> &result();
};

// Room for every logit of a row as a sort key and as a probability: what the
// sampler needs for rows that keep more candidates than its short way holds.
struct SamplerScratch {
    DevTensor keys, probs;      // [max_seqs, cap]
    long long cap = 0;
};

class Engine {
public:
    // max_seqs 0: max(1, min(256, max_tokens / 64))
    Engine(std::unique_ptr<Device> dev, std::unique_ptr<DecoderModel> model, long long max_tokens,
           int max_seqs);
    ~Engine();

    // Reads config.json, picks the model through the registry and loads the
    // folder's safetensors by tensor name.
    static std::unique_ptr<Engine> open(const std::string &model_dir, DType dtype, long long max_tokens,
                                        int max_seqs, int device);
    // The same architecture lookup from a config.json given as text, with weights
    // made at random on the device.
    static std::unique_ptr<Engine> open_random(const Json &config_json, unsigned long long seed, DType dtype,
                                               long long max_tokens, int max_seqs, int device);

    // sequences
    int new_sequence() { return cache->new_sequence(); }
    void free_sequence(int slot);
    long long length(int slot) const;
    bool truncate_sequence(int slot, long long n);

    // Checks a step and lays out its rows; touches nothing.
    struct Plan {
        StepKind kind = PREFILL;
        std::vector<int32_t> tokens;
        std::vector<int> slots;
        std::vector<long long> pos0, lens;
        long long n_rows = 0, n_want = 0;
    };
    Plan plan(const std::vector<StepEntry> &entries) const;

    // Runs the entries' tokens as one batch.  Returns the float32 logits
    // [*n_wanted, vocab] on the device, in the order of the entries and of each
    // entry's want (an empty Buf when nothing is wanted).  The work is queued on
    // the device's stream; the caller synchronizes (or copies on that stream).
    Buf step(const std::vector<StepEntry> &entries, long long *n_wanted);
    // When set, the next steps also leave the residual stream after every entry of
    // the run order here (see StepContext::trace): a tool for finding the first
    // layer that goes wrong, not a product path.
    std::vector<std::vector<float>> *trace = nullptr;

    // One decode step for sequences that each go on by one token, with the choice
    // of the next token on the device.  decode_begin launches and returns at once;
    // with tokens null the sequences go on from the tokens chosen by the step begun
    // last, which must have had the same slots in the same order (only when
    // decodes_ahead()).  Steps end in the order in which they began, and at most
    // two may be under way.  sampled: the slots' sampler settings apply (else every
    // row takes its first maximum); long_way: some row may keep more candidates
    // than the sampler's short way holds.
    bool decodes_ahead() const { return use_graphs; }
    PendingDecode *decode_begin(const std::vector<int> &slots, const int32_t *tokens, bool sampled,
                                bool long_way);
    const std::vector<int32_t> &decode_end(PendingDecode *p) { return p->result(); }

    // One token per row of logits [rows, vocab] (on the device), chosen on the
    // device by the slots' settings; the tokens on the host.  forced (may be null):
    // how many draws had one candidate only.
    std::vector<int32_t> pick(const float *logits, const std::vector<int> &slots, bool sampled,
                              bool long_way, int *forced);

    SamplerScratch &sampler_scratch();
    // Whether a request with these settings needs the sampler's long way.
    bool needs_long_way(float temperature, int top_k) const;

    // Throws Error(JB_LLM_EFAIL) when a bounded wait of a tensor-core kernel ran
    // out since the last call (its output was not valid).  Synchronizes.
    void check_device_errors();

    Json describe() const;
    size_t n_graphs() const { return graphs_.size(); }
    // Waits for the device and lets go of every captured decode step.
    void drop_graphs();

    std::unique_ptr<Device> dev;
    std::unique_ptr<DecoderModel> model;
    std::unique_ptr<Cache> cache;
    std::unique_ptr<ArchConfig> config;     // null for a model built from a spec
    DType dtype;
    long long max_positions;
    bool use_graphs;
    size_t max_graphs = 64;
    long long graph_captures = 0;           // how many decode steps have been captured

private:
    friend class DecodeGraph;
    std::vector<LayerCache> layer_caches(const std::map<const KVGroup *, std::pair<const int32_t *, int>> &bt);
    // captured decode steps by (batch, context bound, sampled, long way); the one
    // used last at the back, the oldest goes when there are more than max_graphs
    using GraphKey = std::tuple<int, long long, bool, bool>;
    std::list<std::pair<GraphKey, std::unique_ptr<DecodeGraph>>> graphs_;
    DecodeGraph *last_graph_ = nullptr;     // the graph of the decode step begun last
    std::vector<int> last_slots_;
    std::vector<int> cache_entry_;          // run-order entry -> entry whose cache it uses, or -1
    std::unique_ptr<SamplerScratch> sampler_scratch_;
    PendingDecode eager_pending_;
};

}  // namespace jb
