#include "graph.h"

#include <cstring>

namespace jb {

DecodeGraph::DecodeGraph(Engine &e, int batch, long long bound, bool sampled, bool long_way)
    : eng_(e), batch_(batch), bound_(bound), sampled_(sampled), long_way_(long_way) {
    width_ = (int)((pages_for(bound) + 7) / 8 * 8);
    size_t n_groups = e.cache->groups.size();
    total_ = 4 * (size_t)batch + n_groups * (size_t)batch * (size_t)width_;
    for (int i = 0; i < 2; i++) {
        cuda_check(cudaMallocHost((void **)&host_[i], total_ * 4), "pinned host allocation");
        memset(host_[i], 0, total_ * 4);
        cuda_check(cudaMallocHost((void **)&out_host_[i], (size_t)batch * 4), "pinned host allocation");
        cuda_check(cudaEventCreateWithFlags(&events_[i], cudaEventDisableTiming), "cudaEventCreate");
    }
    dev_ = e.dev->tensor(I32, {(long long)total_}, true);
}

DecodeGraph::~DecodeGraph() {
    if (exec_) cudaGraphExecDestroy(exec_);
    if (graph_) cudaGraphDestroy(graph_);
    for (int i = 0; i < 2; i++) {
        if (events_[i]) cudaEventDestroy(events_[i]);
        if (host_[i]) cudaFreeHost(host_[i]);
        if (out_host_[i]) cudaFreeHost(out_host_[i]);
    }
}

void DecodeGraph::launch(bool capturing) {
    Engine &e = eng_;
    int B = batch_;
    int32_t *d = (int32_t *)dev_.ptr;
    StepContext ctx;
    ctx.kind = DECODE;
    ctx.dtype = e.dtype;
    ctx.dev = e.dev.get();
    ctx.n_rows = B;
    ctx.n_seqs = B;
    ctx.hidden = e.model->spec.hidden_size;
    ctx.row_pos = d + B;
    ctx.row_seq = d + 2 * B;
    ctx.seq_slot = d + 3 * B;
    ctx.max_pos = bound_ - 1;
    ctx.captured = capturing;
    std::map<const KVGroup *, std::pair<const int32_t *, int>> bt;
    for (size_t gi = 0; gi < e.cache->groups.size(); gi++)
        bt[e.cache->groups[gi].get()] = {d + 4 * (size_t)B + gi * (size_t)B * (size_t)width_, width_};
    std::vector<LayerCache> caches = e.layer_caches(bt);
    Buf logits = e.model->forward(ctx, d, caches, nullptr, -1);
    // the chosen tokens take the place of the tokens the step was fed
    ops::SamplerArrays s;
    if (sampled_) {
        Cache &c = *e.cache;
        s.row_slot = d + 3 * B;
        s.temperature = (const float *)c.temperature.ptr;
        s.top_k = (const int32_t *)c.top_k.ptr;
        s.top_p = (const float *)c.top_p.ptr;
        s.min_p = (const float *)c.min_p.ptr;
        s.rng = (unsigned long long *)c.rng.ptr;
        if (long_way_) {
            SamplerScratch &sc = e.sampler_scratch();
            s.big_keys = (unsigned long long *)sc.keys.ptr;
            s.big_probs = (float *)sc.probs.ptr;
            s.big_cap = sc.cap;
        }
    }
    ops::sample(*e.dev, logits.as<float>(), B, (int)e.model->spec.vocab_size, s, d);
}

PendingDecode *DecodeGraph::begin(const std::vector<int> &slots, const int32_t *tokens,
                                  const std::vector<long long> &pos0, DecodeGraph *before) {
    Engine &e = eng_;
    Device &dv = *e.dev;
    int B = batch_;
    int turn = turn_;
    turn_ = 1 - turn;
    // the buffers of this turn were last used two steps ago: that step has to be
    // over, and its tokens taken, before they are written again
    if (used_[turn]) pending_[turn].result();
    int32_t *h = host_[turn];
    if (tokens) memcpy(h, tokens, (size_t)B * 4);
    for (int i = 0; i < B; i++) {
        h[B + i] = (int32_t)pos0[(size_t)i];
        h[2 * B + i] = i;
        h[3 * B + i] = slots[(size_t)i];
    }
    for (size_t gi = 0; gi < e.cache->groups.size(); gi++)
        e.cache->block_table(*e.cache->groups[gi], slots, width_, h + 4 * (size_t)B + gi * (size_t)B * (size_t)width_);
    int32_t *d = (int32_t *)dev_.ptr;
    if (sampled_ && long_way_) e.sampler_scratch();      // allocated before any capture
    if (tokens) {
        cuda_check(cudaMemcpyAsync(d, h, total_ * 4, cudaMemcpyHostToDevice, dv.stream), "copy to the device");
        dv.h2d_bytes += (long long)total_ * 4;
    } else {
        if (before && before != this)
            cuda_check(cudaMemcpyAsync(d, before->dev_.ptr, (size_t)B * 4, cudaMemcpyDeviceToDevice, dv.stream),
                       "copy on the device");
        cuda_check(cudaMemcpyAsync(d + B, h + B, (total_ - (size_t)B) * 4, cudaMemcpyHostToDevice, dv.stream),
                   "copy to the device");
        dv.h2d_bytes += (long long)(total_ - (size_t)B) * 4;
    }
    if (!exec_) {
        // the first step runs eagerly (it brings every temporary into the pool and is
        // a real step); the capture that follows records without running
        launch(false);
        cuda_check(cudaMemcpyAsync(out_host_[turn], d, (size_t)B * 4, cudaMemcpyDeviceToHost, dv.stream),
                   "reading the chosen tokens");
        cuda_check(cudaEventRecord(events_[turn], dv.stream), "cudaEventRecord");
        dv.sync();
        long long before_n = ops::launches();
        cuda_check(cudaStreamBeginCapture(dv.stream, cudaStreamCaptureModeRelaxed), "cudaStreamBeginCapture");
        cudaGraph_t g = nullptr;
        try {
            launch(true);
        } catch (...) {
            cudaStreamEndCapture(dv.stream, &g);
            if (g) cudaGraphDestroy(g);
            cudaGetLastError();
            throw;
        }
        cuda_check(cudaStreamEndCapture(dv.stream, &g), "cudaStreamEndCapture");
        graph_ = g;
        cuda_check(cudaGraphInstantiate(&exec_, graph_, 0), "cudaGraphInstantiate");
        kernels = (int)(ops::launches() - before_n);
        ops::count_launches(-(long long)kernels);       // recorded, not run
        e.graph_captures++;
    } else {
        cuda_check(cudaGraphLaunch(exec_, dv.stream), "cudaGraphLaunch");
        ops::count_launches(kernels);
        cuda_check(cudaMemcpyAsync(out_host_[turn], d, (size_t)B * 4, cudaMemcpyDeviceToHost, dv.stream),
                   "reading the chosen tokens");
        cuda_check(cudaEventRecord(events_[turn], dv.stream), "cudaEventRecord");
    }
    pending_[turn] = PendingDecode();
    pending_[turn].event = events_[turn];
    pending_[turn].n = B;
    pending_[turn].out_host = out_host_[turn];
    used_[turn] = true;
    return &pending_[turn];
}

}  // namespace jb
