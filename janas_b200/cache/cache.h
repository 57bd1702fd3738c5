// The cache: paged keys and values per layer group, and per-sequence state.
//
// A sequence lives in a *slot*.  The slot records how many tokens of the sequence
// have been computed and owns, in every layer group, the pages that hold its keys
// and values.  A page is PAGE positions of all KV heads of one layer; a group is
// the set of run-order entries whose mixers need the same kind of storage (the
// same number of KV heads and head size, and either all positions or a window of
// them).  Every group has a pool and tensors of its own:
//
//     K, V: [entries of the group, pages, kv_heads, PAGE, head_dim]
//
// A group with a window gives pages back as soon as no later token can see them,
// so a long sequence holds only about window / PAGE + 1 pages there.
//
// Beside the pages, every slot has state of fixed size: the sampler's settings and
// random state, and whatever fixed-size tensors the model's mixers ask for
// (StateSpec); these are zeroed when a slot is taken.  Qwen3 asks for none.
//
// The reference keeps the same things per sequence in struct janas_seq
// (src/llm/model_impl.h:128-171: keys, values, recurrent state), describes layer
// groups by per-group geometry arrays (src/llm/model_impl.h:262-274, filled in
// src/llm/model_load.c:1113-1146) and reuses a server slot for the next request
// (src/server/engine.c:826-838,885-891).
//
// Both pools fail loudly on misuse (a page or slot freed twice, or one that was
// never handed out), because a page held by two sequences is a silent corruption
// that would only show as wrong tokens much later.
#pragma once

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../core/error.h"
#include "../core/json.h"
#include "../engine/device.h"

namespace jb {

constexpr int PAGE = 64;    // positions per page; the kernels use the same number (jb_page())

// No free page or slot is left (the reference's JANAS_LLM_EFULL, include/janas/llm.h:43-53).
struct CacheFull : Error {
    explicit CacheFull(const std::string &m) : Error(JB_LLM_EFULL, m) {}
};

inline long long pages_for(long long n_tokens) { return (n_tokens + PAGE - 1) / PAGE; }

// The pages of one layer group.  Pages are handed out lowest-free first and come
// back when a sequence ends or a window has moved past them.
class PagePool {
public:
    PagePool(int n_pages, std::string name);
    int n_pages() const { return n_pages_; }
    int n_free() const { return (int)free_.size(); }
    std::vector<int> take(int count);                 // CacheFull, and then nothing is taken
    void give_back(const std::vector<int> &pages);    // Error when one is not held
    void check() const;                               // Error when a page is lost or free twice

private:
    int n_pages_;
    std::string name_;
    std::vector<int> free_;
    std::vector<char> held_;
};

// The slots: one per live sequence.
class SlotPool {
public:
    explicit SlotPool(int n_slots);
    int n_slots() const { return n_slots_; }
    int n_free() const { return (int)free_.size(); }
    bool live(int slot) const { return slot >= 0 && slot < n_slots_ && live_[(size_t)slot]; }
    int take();                                       // CacheFull
    void give_back(int slot);                         // Error when it is not in use
    void check() const;

private:
    int n_slots_;
    std::vector<int> free_;
    std::vector<char> live_;
};

// What a mixer needs stored per position.  window 0: every position stays;
// otherwise only the last `window` positions can be read again.
struct KVSpec {
    int num_kv_heads = 0, head_dim = 0, window = 0;
    bool none() const { return num_kv_heads == 0; }
    bool operator==(const KVSpec &o) const {
        return num_kv_heads == o.num_kv_heads && head_dim == o.head_dim && window == o.window;
    }
};

// Fixed-size state a mixer keeps per sequence: a tensor of this shape, zero at
// the sequence's start.  An empty shape: none.
struct StateSpec {
    std::vector<long long> shape;
    DType dtype = F32;
    bool none() const { return shape.empty(); }
    size_t bytes() const { size_t n = dtype_size(dtype); for (auto s : shape) n *= (size_t)s; return n; }
};

// The storage of one layer group.
class KVGroup {
public:
    KVGroup(KVSpec spec, std::vector<int> entries, int n_pages, int n_slots);
    KVSpec spec;
    std::vector<int> entries;              // run-order entries stored here
    std::map<int, int> index;              // entry -> place within the group
    PagePool pool;
    DevTensor k, v;                        // empty when the cache holds bookkeeping only
    // per slot: the page of every page index (absolute position / PAGE), -1 once released
    std::vector<std::vector<int>> pages;

    size_t entry_bytes() const;            // bytes of one entry's K (or V)
    void *k_of(int entry) const { return (char *)k.ptr + (size_t)index.at(entry) * entry_bytes(); }
    void *v_of(int entry) const { return (char *)v.ptr + (size_t)index.at(entry) * entry_bytes(); }
    int first_needed_page(long long next_pos) const;
    void extend(int slot, long long end);
    void release_unseen(int slot, long long next_pos);
    void free_slot(int slot);
    int held(int slot) const;
};

// Sampling settings of one sequence, as they lie in the slot's state.
struct SamplerSettings {
    unsigned long long seed = 0;
    float temperature = 0;
    int top_k = 0;
    float top_p = 0, min_p = 0;
};

class Cache {
public:
    // kv_specs[e] / state_specs[e]: what run-order entry e needs (none() for
    // nothing; entries that read another entry's cache have none).  max_tokens:
    // the most tokens that live sequences may hold at one time, each sequence's
    // count rounded up to a multiple of PAGE; max_seqs: the most sequences alive
    // at one time.  dev null: bookkeeping only, no storage (for tests of the
    // decisions on a machine without a GPU).
    Cache(const std::vector<KVSpec> &kv_specs, const std::vector<StateSpec> &state_specs,
          long long max_tokens, int max_seqs, DType dtype, Device *dev);

    // sequences
    int new_sequence();
    void free_sequence(int slot);
    long long length(int slot) const { return length_.at((size_t)slot); }
    bool can_truncate(int slot, long long n) const;
    bool truncate(int slot, long long n);
    void set_samplers(const std::vector<int> &slots, const std::vector<SamplerSettings> &s);
    // Slots whose settings were never set since they were taken get the defaults
    // (greedy): the device's arrays may still hold an earlier sequence's.
    void ensure_samplers(const std::vector<int> &slots);
    const SamplerSettings &sampler(int slot) const { return sampler_of_.at((size_t)slot); }

    // steps
    void reserve(const std::vector<int> &slots, const std::vector<long long> &counts);
    void advance(const std::vector<int> &slots, const std::vector<long long> &counts);
    // int32 [len(slots), width]: the page of every page index of each slot (-1 where
    // there is none); width() is a multiple of 8
    int table_width(const KVGroup &g, const std::vector<int> &slots) const;
    void block_table(const KVGroup &g, const std::vector<int> &slots, int width, int32_t *out) const;

    // checks
    long long tokens_held() const;
    size_t bytes() const;
    void check() const;
    Json describe() const;

    Device *dev;
    DType dtype;
    long long max_tokens;
    int max_seqs;
    SlotPool slots;
    std::vector<std::unique_ptr<KVGroup>> groups;
    std::map<int, KVGroup *> group_of;             // entry -> its group
    // fixed-size state per slot, on the device
    DevTensor rng, temperature, top_k, top_p, min_p;
    std::map<int, DevTensor> mixer_state;          // entry -> [max_seqs, *shape]
    std::map<int, StateSpec> state_spec;

private:
    std::vector<long long> length_;
    std::vector<SamplerSettings> sampler_of_;      // the host's copy of each slot's settings
    std::vector<char> sampler_set_;
    void zero_state(int slot);
};

}  // namespace jb
