// The interfaces of the parts a layer is put together from, and their registry.
//
// A part is built from a PartSpec (its registered kind and its constants), the
// compute dtype and the device.  It says which tensors it needs below a name
// prefix (tensors), takes them (load) and computes (apply / forward).  No part
// knows which model it is in: sizes and constants arrive as parameters,
// everything about the current step arrives in a StepContext.
//
// Outputs of mixers and feed-forwards are *stacks of partial sums*: float32
// [S, n, hidden] whose sum over S is the part's output (S = 1 unless a matrix
// product was split over its inner dimension).  The block adds them to the
// residual stream in the order 0 .. S-1.
//
// A new mixer, feed-forward, norm, position encoding or block arrangement is a
// class registered under a new name (register_part / register_block); a
// configuration then refers to it by that name in a PartSpec.  Nothing else in
// the library has to change.  Parts can also be registered from outside the
// library through the C interface (parts/foreign.cpp): a callback that answers
// the same questions.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../cache/cache.h"
#include "../config/spec.h"
#include "../csrc/launch.h"
#include "../weights/loader.h"

namespace jb {

enum StepKind {
    PREFILL,   // every sequence starts at its first token
    DECODE,    // every sequence goes on by one token
    EXTEND     // anything else (tokens appended to sequences that have some)
};
const char *step_kind_name(StepKind k);

// What a mixer sees of the cache for the run-order entry it runs as.
struct LayerCache {
    ops::AttnCache kv;                  // this entry's K/V pages and the step's block table
    int kv_heads = 0, head_dim = 0;
    void *state = nullptr;              // [slots, *state shape], indexed by slot; or null
    StateSpec state_spec;
    int n_slots = 0;
};

// One step: the rows (tokens) it runs and where each belongs.  Rows are the
// sequences' tokens one sequence after the other.  row_pos, row_seq and seq_slot
// are int32 arrays on the device; the seq_* vectors are on the host and empty in
// a captured decode step (which is replayed with other contents).
struct StepContext {
    StepKind kind = PREFILL;
    DType dtype = BF16;
    Device *dev = nullptr;
    long long n_rows = 0;
    int n_seqs = 0;
    long long hidden = 0;                // width of the residual stream
    const int32_t *row_pos = nullptr;    // position of each row in its sequence
    const int32_t *row_seq = nullptr;    // index of the row's sequence within the step
    const int32_t *seq_slot = nullptr;   // slot of each sequence
    std::vector<int> seq_slots;
    std::vector<long long> seq_pos0;     // tokens each sequence had before the step
    std::vector<long long> seq_len;      // tokens each sequence brings
    std::vector<long long> seq_row0;     // first row of each sequence (n_seqs + 1 values)
    long long max_pos = 0;               // the largest position of any row (a bound, in a captured step)
    bool captured = false;               // the launches are being recorded into a graph
    // For finding the first layer that goes wrong: when set, the model copies the
    // residual stream [n_rows, hidden] to the host after every entry of the run
    // order (what is still to be added is added first), one vector per entry.
    std::vector<std::vector<float>> *trace = nullptr;
    // what a part computed once for all layers of this step (the attention's blocks)
    struct Extra { Buf buf; int n = 0; };
    std::map<std::string, Extra> extras;
};

using TensorMap = std::map<std::string, DevTensor>;

class Part {
public:
    Part(const PartSpec &s, DType dt, Device *d) : spec(s), dtype(dt), dev(d) {}
    virtual ~Part() = default;
    // name -> TensorSpec of every tensor this part reads, below prefix (which ends
    // without a dot; an empty prefix means no prefix); appended to out
    virtual void tensors(const std::string &prefix, TensorList &out) const {}
    // Takes its tensors (on the device, in their resident dtype) out of the map.
    virtual void load(const std::string &prefix, TensorMap &t) {}
    virtual size_t weight_bytes() const { return 0; }
    virtual Json info() const { return Json::object(); }

    PartSpec spec;
    DType dtype;
    Device *dev;

    static std::string name(const std::string &prefix, const std::string &leaf) {
        return prefix.empty() ? leaf : prefix + "." + leaf;
    }
    // the tensor `name` out of the map (it is erased there); Error when it is missing
    static DevTensor take(TensorMap &t, const std::string &name);
};

class Norm : public Part {
public:
    using Part::Part;
    // Normalizes the rows of the float32 residual stream x [n, size].  With delta
    // (a stack of partial sums) x += sum(delta) happens first, in place.  With
    // rows (n_out indices on the device) only those rows are normalized and
    // returned.  The result is [n or n_out, size] in out_dt.
    virtual Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta,
                      const int32_t *rows, long long n_out) = 0;
    virtual long long size() const = 0;
};

class PositionEncoding : public Part {
public:
    using Part::Part;
    // Called once the cache's size is known: positions below n will be asked for.
    virtual void prepare(long long n_positions) {}
    virtual const float *cos() const { return nullptr; }     // [n_positions, rotary_dim / 2] or null
    virtual const float *sin() const { return nullptr; }
    virtual int rotary_dim() const { return 0; }
    virtual long long n_positions() const { return 1ll << 62; }
};

class Mixer : public Part {
public:
    using Part::Part;
    // Keys and values per position that the cache should hold (none() for nothing).
    virtual KVSpec kv_spec() const { return KVSpec(); }
    // Fixed-size state per sequence (none() for nothing).
    virtual StateSpec state_spec() const { return StateSpec(); }
    virtual void prepare(long long n_positions) {}
    // Whether the mixer can run a step of this kind.
    virtual bool supports(StepKind kind) const { return true; }
    // True when forward() reads everything that changes between decode steps
    // (positions, slots, block tables) from the context's device arrays only, so
    // that a captured decode step can be replayed with new contents.
    virtual bool graph_safe() const { return false; }
    // h: [n, hidden] in the compute dtype -> stack [S, n, hidden] float32
    virtual Stack forward(StepContext &ctx, const void *h, LayerCache &cache) = 0;
};

class FeedForward : public Part {
public:
    using Part::Part;
    virtual bool graph_safe() const { return true; }
    virtual Stack forward(StepContext &ctx, const void *h) = 0;
};

// The arrangement of one layer's parts around the residual stream.
class Block {
public:
    Block(std::unique_ptr<Mixer> m, std::unique_ptr<FeedForward> f, std::unique_ptr<Norm> n1,
          std::unique_ptr<Norm> n2)
        : mixer(std::move(m)), feed_forward(std::move(f)), mixer_norm(std::move(n1)),
          ffn_norm(std::move(n2)) {}
    virtual ~Block() = default;
    // x: the float32 residual stream [n, hidden], updated in place; pending: a
    // stack of partial sums not yet added to x (empty for none), replaced by what
    // this layer leaves to be added.
    virtual void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) = 0;

    std::unique_ptr<Mixer> mixer;
    std::unique_ptr<FeedForward> feed_forward;
    std::unique_ptr<Norm> mixer_norm, ffn_norm;
};

// ------------------------------------------------------------------ registry
using PartFactory = std::function<std::unique_ptr<Part>(const PartSpec &, DType, Device *)>;
using BlockFactory = std::function<std::unique_ptr<Block>(
    std::unique_ptr<Mixer>, std::unique_ptr<FeedForward>, std::unique_ptr<Norm>, std::unique_ptr<Norm>)>;

// role: "mixer", "feed_forward", "norm" or "position"
void register_part(const std::string &role, const std::string &kind, PartFactory f);
void register_block(const std::string &kind, BlockFactory f);
std::vector<std::string> registered_parts(const std::string &role);

std::unique_ptr<Part> build_part(const std::string &role, const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<Mixer> build_mixer(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<FeedForward> build_feed_forward(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<Norm> build_norm(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<PositionEncoding> build_position(const PartSpec &spec, DType dt, Device *dev);
std::unique_ptr<Block> build_block(const std::string &kind, std::unique_ptr<Mixer> m,
                                   std::unique_ptr<FeedForward> f, std::unique_ptr<Norm> n1,
                                   std::unique_ptr<Norm> n2);

// Several matrices over the same input as one, rows one after the other, so that
// one product serves them all (the reference dispatches q, k, v as one group and
// gate, up as one: src/llm/model_attn.c:255, src/llm/model_ffn.c:349).  If their
// dtypes differ, the widest is taken.  The sources are released as they are copied.
DevTensor fuse_rows(Device &dev, std::vector<DevTensor> &mats);

// the built-in kinds (each file registers its own)
void register_builtin_norms();
void register_builtin_positions();
void register_builtin_mixers();
void register_builtin_feed_forwards();
void register_builtin_blocks();

}  // namespace jb

// csrc/convert.cu: element type conversions on the device (bfloat16 <-> float32)
extern "C" int jb_convert(const void *src, int src_dt, void *dst, int dst_dt, long long n,
                          cudaStream_t st);
