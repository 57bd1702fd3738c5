// The one generic decoder: embedding, the layers in run order, final norm, head.
//
// It is built from a ModelSpec alone.  For every layer the spec names the block
// arrangement, the mixer, the feed-forward and the norms; the classes come from
// the part registries.  run_order is walked entry by entry; an entry names the
// layer whose weights run and, optionally, an earlier entry whose cache it reads
// instead of writing one of its own.
//
// The reference's forward pass has the same shape: embedding, layer loop, final
// norm of the rows whose logits are wanted, head (src/llm/model.c:647-876; the
// head is the embedding table when the file has no output matrix:
// src/llm/model_load.c:1004-1007).
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "../parts/part.h"

namespace jb {

class DecoderModel {
public:
    // dev may be null: the model can then list its tensors but not load or run.
    DecoderModel(const ModelSpec &spec, DType dtype, Device *dev);

    // Every tensor the model reads, by checkpoint name, in the model's order.
    TensorList tensors() const;
    // The tensors of layer i alone (its four parts), and of what is not a layer.
    TensorList layer_tensors(int i) const;
    TensorList top_tensors() const;

    // Loading goes piece by piece so that at no time more than one layer's tensors
    // lie on the device twice (as they came and fused): first load_top, then
    // load_layer for every layer.  Each takes its tensors out of the map.
    void load_top(TensorMap &t);
    void load_layer(int i, TensorMap &t);
    // From a checkpoint (checked against tensors() first) or at random.
    void load_checkpoint(const Checkpoint &ckpt);
    void load_random(unsigned long long seed);

    // Bytes of weights a step reads once (the embedding table counts only as the
    // head, when tied; else only a few rows of it are read).
    size_t weight_bytes() const;

    std::vector<KVSpec> kv_specs() const;         // per run-order entry
    std::vector<StateSpec> state_specs() const;
    void prepare(long long n_positions);
    bool supports(StepKind kind) const;
    bool graph_safe() const;

    // tokens: int32 [n] on the device; caches[e]: the cache view of run-order entry
    // e; want_rows: n_want int32 row indices on the device whose logits are wanted
    // (null with n_want < 0: all rows; n_want == 0: none).  Returns float32
    // [wanted, vocab] (an empty Buf when nothing is wanted).
    Buf forward(StepContext &ctx, const int32_t *tokens, std::vector<LayerCache> &caches,
                const int32_t *want_rows, long long n_want);

    ModelSpec spec;
    DType dtype;
    Device *dev;
    std::vector<std::unique_ptr<Block>> blocks;
    std::unique_ptr<Norm> final_norm;
    DevTensor embedding, head;
    bool loaded = false;

private:
    void layer_names(int i, std::string n[4]) const;
};

}  // namespace jb
