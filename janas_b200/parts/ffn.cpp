// The SwiGLU feed-forward: down(SiLU(gate(x)) * up(x)), no biases
// (src/llm/model_ffn.c:147-154, src/llm/vmath.h:64-68).  The reference runs a
// dense layer as the single expert of a mixture with router weight exactly 1
// (src/llm/model_load.c:505-514); here it is a part of its own.
#include "part.h"

namespace jb {

namespace {

// params: hidden_size, intermediate_size
class SwiGLU : public FeedForward {
public:
    // Rows from which gate, up and the activation run as one kernel.  Measured on
    // B200 at Qwen3-4B sizes: 167 against 165 + 37 microseconds at 2,048 rows, 103
    // against 109 at 1,024, even at 512; with few rows the one kernel cannot cut k
    // into parts and loses (29 against 20 at 8 rows).
    static constexpr long long FUSED_FROM = 512;
    // Rows up to which the one kernel runs too, in tiles of 64 gate and 64 up
    // features, if the plain product would not cut k either (a wide feed-forward:
    // the tiles alone fill the SMs).  It saves the activation kernel of a decode step
    // and of a short prompt (a prompt of 128 tokens: 3.22 -> 3.13 ms).
    static constexpr long long FUSED_UP_TO = 128;

    SwiGLU(const PartSpec &s, DType dt, Device *d) : FeedForward(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        inter_ = s.get_int("intermediate_size");
        if (hidden_ <= 0 || inter_ <= 0) config_error("swiglu: sizes must be positive");
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, "gate_proj.weight"), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, "up_proj.weight"), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, "down_proj.weight"), TensorSpec{{hidden_, inter_}, MATRIX, false});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        std::vector<DevTensor> gu = {take(t, name(prefix, "gate_proj.weight")),
                                     take(t, name(prefix, "up_proj.weight"))};
        w_gate_up_ = fuse_rows(*dev, gu);
        w_down_ = take(t, name(prefix, "down_proj.weight"));
    }

    size_t weight_bytes() const override { return w_gate_up_.bytes() + w_down_.bytes(); }

    Stack forward(StepContext &ctx, const void *h) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        Buf act;
        fused_last_ = false;
        if (ctx.dtype == BF16 &&
            (n >= FUSED_FROM || (n <= FUSED_UP_TO && ops::linear_parts(n, 2 * inter_, hidden_) == 1))) {
            // enough rows, or enough features, to fill the SMs without cutting k:
            // gate, up and the activation in one kernel
            act = ops::linear_swiglu(d, h, ctx.dtype, n, hidden_, w_gate_up_);
            fused_last_ = (bool)act;
        }
        if (!act) {
            Stack gu = ops::linear(d, h, ctx.dtype, n, hidden_, w_gate_up_);
            act = ops::swiglu(d, gu, ctx.dtype);
        }
        return ops::linear(d, act.ptr, ctx.dtype, n, inter_, w_down_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("fused_from", FUSED_FROM);
        o.set("fused_up_to", FUSED_UP_TO);
        o.set("fused_last", fused_last_);
        return o;
    }

private:
    long long hidden_, inter_;
    DevTensor w_gate_up_, w_down_;
    bool fused_last_ = false;      // whether the last forward took the one-kernel way
};

}  // namespace

void register_builtin_feed_forwards() {
    register_part("feed_forward", "swiglu", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new SwiGLU(s, dt, d));
    });
}

}  // namespace jb
