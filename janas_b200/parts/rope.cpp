// NeoX ("rotate half") rotary position encoding.
//
// theta(p, i) = (float)p * powf(theta, -2 i / rotary_dim), i < rotary_dim / 2; the
// pair (i, i + half) of a head is rotated by it (src/llm/model.c:100-113,
// src/llm/model_attn.c:31-39).  The powers are computed once on the host in double
// and rounded to float, as the reference's powf does (src/llm/jmath.c:131-134);
// the table of cos and sin is filled on the device from double-precision sincos of
// the float angle (src/llm/jmath.c:163-200) when the cache's size is known.
//
// The rotation itself is applied by the attention kernel that also normalizes the
// heads and appends K and V (csrc/rope.cu); this part owns the constants and the
// table.  Only the whole head can be rotated (rotary_dim == head size); the
// reference's partial rotation (n_rot < head size) is not built.
#include <cmath>

#include "part.h"

namespace jb {

namespace {

// params: rotary_dim, theta, max_positions
class RopeNeox : public PositionEncoding {
public:
    RopeNeox(const PartSpec &s, DType dt, Device *d) : PositionEncoding(s, dt, d) {
        rotary_dim_ = (int)s.get_int("rotary_dim");
        theta_ = s.get_double("theta");
        max_positions_ = s.get_int("max_positions");
        if (rotary_dim_ <= 0 || rotary_dim_ % 2) config_error("rope_neox: rotary_dim must be even and positive");
        int half = rotary_dim_ / 2;
        inv_freq_.resize((size_t)half);
        for (int i = 0; i < half; i++) {
            // the exponent in float arithmetic, the power in double, rounded once
            float expo = -2.0f * (float)i / (float)rotary_dim_;
            inv_freq_[(size_t)i] = (float)std::pow((double)(float)theta_, (double)expo);
        }
    }

    void prepare(long long n_positions) override {
        long long n = std::min(n_positions, max_positions_);
        if (n <= n_) return;
        if (!dev) fail(JB_LLM_EFAIL, "rope_neox: no device to fill the table on");
        dev->make_current();
        int half = rotary_dim_ / 2;
        DevTensor inv = dev->tensor(F32, {half});
        cuda_check(cudaMemcpy(inv.ptr, inv_freq_.data(), (size_t)half * 4, cudaMemcpyHostToDevice),
                   "copying the rotation's frequencies");
        DevTensor c = dev->tensor(F32, {n, half}), s = dev->tensor(F32, {n, half});
        ops::rope_table(*dev, (const float *)inv.ptr, half, n, (float *)c.ptr, (float *)s.ptr);
        dev->sync();
        cos_ = c;
        sin_ = s;
        n_ = n;
    }

    const float *cos() const override { return (const float *)cos_.ptr; }
    const float *sin() const override { return (const float *)sin_.ptr; }
    int rotary_dim() const override { return rotary_dim_; }
    long long n_positions() const override { return n_; }

    Json info() const override {
        Json o = Json::object();
        o.set("rotary_dim", rotary_dim_);
        o.set("n_positions", n_);
        o.set("cos", (unsigned long long)(uintptr_t)cos_.ptr);
        o.set("sin", (unsigned long long)(uintptr_t)sin_.ptr);
        return o;
    }

private:
    int rotary_dim_;
    double theta_;
    long long max_positions_;
    std::vector<float> inv_freq_;
    DevTensor cos_, sin_;
    long long n_ = 0;
};

// No position encoding: q and k are used as they are.
class NoPosition : public PositionEncoding {
public:
    using PositionEncoding::PositionEncoding;
};

}  // namespace

void register_builtin_positions() {
    register_part("position", "rope_neox", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new RopeNeox(s, dt, d));
    });
    register_part("position", "none", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new NoPosition(s, dt, d));
    });
}

}  // namespace jb
