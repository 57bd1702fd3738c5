// Block arrangements.  prenorm: x += mixer(norm(x)); x += ffn(norm(x))
// (src/llm/model.c:743-796).
#include "part.h"

namespace jb {

namespace {

class PreNormBlock : public Block {
public:
    using Block::Block;
    void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) override {
        long long n = ctx.n_rows;
        // the add of what the previous part produced is fused into the norm
        Buf h = mixer_norm->apply(ctx, x, n, ctx.dtype, pending ? &pending : nullptr, nullptr, 0);
        Stack d = mixer->forward(ctx, h.ptr, cache);
        h = ffn_norm->apply(ctx, x, n, ctx.dtype, &d, nullptr, 0);
        pending = feed_forward->forward(ctx, h.ptr);
    }
};

}  // namespace

void register_builtin_blocks() {
    register_block("prenorm", [](std::unique_ptr<Mixer> m, std::unique_ptr<FeedForward> f,
                                 std::unique_ptr<Norm> n1, std::unique_ptr<Norm> n2) {
        return std::unique_ptr<Block>(new PreNormBlock(std::move(m), std::move(f), std::move(n1), std::move(n2)));
    });
}

}  // namespace jb
