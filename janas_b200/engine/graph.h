// The decode step of `batch` sequences at positions below `bound`, captured once
// into a CUDA graph and replayed.
//
// All that changes from step to step (tokens, positions, slots, block tables)
// lies in a pinned host buffer that is copied to the device before the graph
// runs; the chosen tokens are written where the next step's tokens are read, so
// a step that goes on from them needs nothing from the host but positions and
// block tables, and can be launched while the step before it runs.  There are
// two pinned buffers each way, used in turn: with at most two steps under way,
// the host never writes what a copy still reads, nor reads what a later step
// may already have written.  Launch sizes that depend on the context (the
// attention's chunk count) are fixed at `bound`; rows whose range is shorter
// leave those chunks at once.
//
// The temporaries of the captured kernels come from the device's pool like any
// step's; their addresses are baked into the graph, which is why the pool keeps
// its memory while graphs exist (engine/device.h).
#pragma once

#include "engine.h"

namespace jb {

class DecodeGraph {
public:
    DecodeGraph(Engine &engine, int batch, long long bound, bool sampled, bool long_way);
    ~DecodeGraph();
    DecodeGraph(const DecodeGraph &) = delete;
    DecodeGraph &operator=(const DecodeGraph &) = delete;

    // Copies the step's inputs, runs the step and copies its tokens back, all on
    // the engine's stream, without waiting.  tokens null: the step is fed what the
    // step begun last chose (`before` is its graph).
    PendingDecode *begin(const std::vector<int> &slots, const int32_t *tokens,
                         const std::vector<long long> &pos0, DecodeGraph *before);

    int kernels = 0;        // kernels per replay

private:
    void launch(bool capturing);
    Engine &eng_;
    int batch_;
    long long bound_;
    bool sampled_, long_way_;
    int width_;
    size_t total_;                      // int32 values of the input buffer
    int32_t *host_[2] = {nullptr, nullptr};
    int32_t *out_host_[2] = {nullptr, nullptr};
    cudaEvent_t events_[2] = {nullptr, nullptr};
    PendingDecode pending_[2];
    bool used_[2] = {false, false};
    int turn_ = 0;
    DevTensor dev_;                     // the device's copy of the inputs; [0, batch) are the tokens
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t exec_ = nullptr;
};

}  // namespace jb
