// The generation loop above the step function, and sessions.
//
// Requests (a prompt, a limit of new tokens, sampling options) are run in batches:
// the prompts of a batch in one step, then one token for every sequence that is
// still going, until all have ended; then the next batch, whose sequences take
// the slots and pages the previous ones gave back.  A sequence ends after a stop
// token (which is part of its output), at its limit of new tokens, or when the
// context is full.  Once a batch has started, no request joins it.
//
// The reference's loop is janas_llm_generate (src/llm/generate.c:1116-1144:
// prompt, then tokens until a stop token or max_new; the stop token is counted:
// :1136-1137; is_stop :699-707; a full context ends the sequence: :895-896) and,
// for several sequences, janas_llm_sessions_step (src/llm/generate.c:1155-1249:
// one pass for all sessions, each token drawn by its own sampler).  Options and
// statistics carry the reference's names (struct janas_gen_options, struct
// janas_gen_stats: src/llm/generate.h:31-86).
//
// The decisions (which requests form a batch, when a sequence ends) are plain host
// code over the Driver interface, so they can be tested with a stand-in for the
// engine on a machine without a GPU.
#pragma once

#include <cstdint>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../cache/cache.h"
#include "../core/error.h"

namespace jb {

constexpr int MAX_STOP = 4;     // JANAS_GEN_MAX_STOP (src/llm/generate.h:27)

enum Finish { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_CONTEXT = 3 };
const char *finish_name(int f);

// Sampling and stopping; all zero: greedy (src/llm/generate.h:31-63).
struct GenOptions {
    int eos = -1;               // stop at this token, -1 for none
    float temperature = 0;      // 0: the most likely token
    int top_k = 0;              // keep the k most likely tokens; 0: no limit
    float top_p = 0;            // keep the most likely tokens up to this mass; 0 or 1: off
    float min_p = 0;            // drop tokens below min_p x the top probability
    unsigned long long seed = 0;
    std::vector<int> stop;      // more stop tokens, besides eos (at most 4)

    void validate() const;      // Error(JB_LLM_EINVAL)
    bool is_stop(int token) const;
    SamplerSettings sampler() const { return SamplerSettings{seed, temperature, top_k, top_p, min_p}; }
};

// Counters of one call (src/llm/generate.h:65-86, the fields that apply).
struct GenStats {
    uint32_t prompt_tokens = 0, new_tokens = 0;
    uint32_t passes = 0;            // forward passes after the prefill
    uint32_t forced_tokens = 0;     // drawn where only one candidate was left
    uint32_t batches = 0;
    double prefill_seconds = 0, decode_seconds = 0, sample_seconds = 0;
    unsigned long long h2d_bytes = 0;   // step inputs copied to the device while decoding
    unsigned long long d2h_bytes = 0;   // chosen tokens read back while decoding
};

struct Request {
    std::vector<int32_t> prompt;
    long long max_new = 0;
    GenOptions options;
};

struct Result {
    std::vector<int32_t> tokens;
    int finish = FINISH_NONE;
};

// ------------------------------------------------------------------ decisions
// Cache tokens a request may come to hold, rounded up to whole pages.  The last
// generated token is never fed back, so it needs no place.
long long tokens_needed(long long prompt_len, long long max_new, long long max_positions);
// Cuts the requests, in their order, into batches of at most max_batch whose
// sequences fit max_tokens of cache together even if every one runs to its limit.
std::vector<std::vector<int>> plan_batches(const std::vector<long long> &prompt_lens,
                                           const std::vector<long long> &max_news, int max_batch,
                                           long long max_tokens, long long max_positions);
// Whether a sequence ends after `token`, its n_generated-th new one; length is
// what the cache holds of it (the token itself not yet).
int finish_reason(int token, long long n_generated, long long max_new, long long length,
                  long long max_positions, const GenOptions &o);
// Whether a sequence goes on after its n_generated-th new token if that is no stop
// token: the next step may then be launched before the token is known.
bool goes_on_unless_stopped(long long n_generated, long long max_new, long long length,
                            long long max_positions);

// ------------------------------------------------------------------ the driver
// One sequence's share of a pass: its next tokens, and whether the token after the
// last of them is to be chosen.
struct FeedEntry {
    int slot = 0;
    const int32_t *tokens = nullptr;
    long long n = 0;
    bool want = false;
};

// What the loop and the sessions need of an engine.
class Driver {
public:
    virtual ~Driver() = default;
    virtual long long vocab_size() const = 0;
    virtual long long max_positions() const = 0;
    virtual int free_slots() const = 0;
    virtual long long free_tokens() const = 0;       // cache tokens no live sequence holds
    virtual int new_sequence() = 0;
    virtual void free_sequence(int slot) = 0;
    virtual long long length(int slot) const = 0;
    virtual bool truncate_sequence(int slot, long long n) = 0;
    virtual void set_samplers(const std::vector<int> &slots, const std::vector<SamplerSettings> &s) = 0;
    virtual bool needs_long_way(float temperature, int top_k) const = 0;
    virtual bool supports_extend() const = 0;
    // One pass over the entries; the chosen token of every entry that wants one, in
    // the entries' order.
    virtual std::vector<int32_t> run(const std::vector<FeedEntry> &entries, bool sampled, bool long_way,
                                     int *forced) = 0;
    // Decode steps that may be queued one ahead (see Engine::decode_begin).
    virtual bool decodes_ahead() const { return false; }
    virtual void *decode_begin(const std::vector<int> &slots, const int32_t *tokens, bool sampled,
                               bool long_way) { return nullptr; }
    virtual std::vector<int32_t> decode_end(void *pending) { return {}; }
    virtual unsigned long long h2d_bytes() const { return 0; }
    // Called where the host has the tokens anyway: throws when the device reported a failure.
    virtual void check_errors() {}
};

class Engine;
std::unique_ptr<Driver> engine_driver(Engine &e);

// Runs all requests; returns their new tokens and why each ended.
std::vector<Result> generate(Driver &d, const std::vector<Request> &requests, int max_batch, GenStats *stats);

// ------------------------------------------------------------------ sessions
// One token sequence that grows by appending tokens (a prompt, a user's turn) and
// by generating them, token by token on request.  Every token is computed once: a
// new turn goes on from the position reached, with the cache kept
// (src/llm/generate.h:88-98).  The names and meanings are those of the reference's
// session interface: append (src/llm/generate.c:709-742), prefill (:744-773: all
// appended tokens but the last, which the next pass takes), next (:886-900: the
// next token, appended to the sequence; status 1 when the context is full, an error
// for an empty sequence), truncate (src/llm/generate.h:160-167), reset,
// set_options (the seed restarts the random sequence, src/llm/generate.h:116-119),
// computed / length / tokens (:166-175), and sessions_step for several sessions on
// one model (src/llm/generate.c:1155-1249).  A session does not stop by itself at a
// stop token: the caller sees every token and decides.
class Session {
public:
    Session(Driver &d, const GenOptions &o);
    ~Session();
    Session(const Session &) = delete;
    Session &operator=(const Session &) = delete;

    long long computed() const;                 // tokens of the sequence the model has computed
    long long length() const { return (long long)hist.size(); }
    void set_options(const GenOptions &o);
    void append(const int32_t *tokens, long long n);
    void truncate(long long n);
    void reset() { truncate(0); }
    void close();
    void prefill();
    // 0 and the token, or 1 when the context is full
    int next(int32_t *token);

    Driver &driver;
    std::vector<int32_t> hist;
    GenOptions options;
    GenStats stats;
    int slot = -1;
};

// Moves several sessions of one driver on together: each one's appended tokens and
// its next token in one pass.  tokens[i], status[i] as Session::next gives them.
void sessions_step(Driver &d, const std::vector<Session *> &sessions, int32_t *tokens, int *status);

}  // namespace jb
