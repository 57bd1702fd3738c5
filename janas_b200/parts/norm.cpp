// RMSNorm: out = (x * 1/sqrt(mean(x^2) + eps)) * w
// (src/llm/model_impl.h:635-644).  The weight is used as it is, not as 1 + w.
#include "part.h"

namespace jb {

namespace {

// params: size, eps
class RMSNorm : public Norm {
public:
    RMSNorm(const PartSpec &s, DType dt, Device *d) : Norm(s, dt, d) {
        size_ = s.get_int("size");
        eps_ = (float)s.get_double("eps");
        if (size_ <= 0) config_error("rmsnorm: size must be positive");
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, "weight"), TensorSpec{{size_}, NORM, false});
    }

    void load(const std::string &prefix, TensorMap &t) override { weight_ = take(t, name(prefix, "weight")); }

    size_t weight_bytes() const override { return weight_.bytes(); }

    Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta,
              const int32_t *rows, long long n_out) override {
        return ops::rmsnorm(*ctx.dev, x, n, size_, weight_, eps_, out_dt, delta, rows, n_out);
    }

    long long size() const override { return size_; }

    Json info() const override {
        Json o = Json::object();
        o.set("size", size_);
        o.set("eps", (double)eps_);
        o.set("weight_dtype", dtype_name(weight_.dt));
        return o;
    }

private:
    long long size_;
    float eps_;
    DevTensor weight_;
};

}  // namespace

void register_builtin_norms() {
    register_part("norm", "rmsnorm", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new RMSNorm(s, dt, d));
    });
}

}  // namespace jb
