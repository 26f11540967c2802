// Root-mean-square norm with a learned scale.
#include "args.h"
#include "../engine/ops.h"

namespace vmb {

// y = x / sqrt(mean(x^2) + eps) * weight, statistics in float32 (src/cpu/ops/rmsnorm.cpp:42-59).  The residual add that
// precedes a norm in a pre-norm block is fused into the same kernel.
class RMSNorm : public Norm {
public:
    RMSNorm(int size, float eps) : size_(size), eps_(eps) {}
    WeightTable weight_specs() const override {
        WeightSpec s;
        s.shape = {size_};
        s.init_ones = true;
        return {{"weight", s}};
    }
    void bind(const Weights& w, BindContext& bc) override { weight_ = bc.upload(w.at("weight"), DType::F32); }   // exact for BF16 and F32 storage
    bool graph_safe() const override { return true; }
    bool as_rms(const float** weight, float* eps) const override {
        *weight = static_cast<const float*>(weight_.ptr);
        *eps = eps_;
        return true;
    }
    void forward(StepContext& ctx, float* h, const void* delta, void* out, const int* rows, int n_rows) override {
        ops::add_rmsnorm(h, delta, static_cast<const float*>(weight_.ptr), eps_, out, rows, rows ? n_rows : ctx.T, size_, ctx.act_dtype, ctx.stream);
    }

private:
    int size_;
    float eps_;
    DeviceTensor weight_;
};

namespace {
RegisterPart reg("norm", "rmsnorm", [](const json::Value& a) {
    return std::make_shared<RMSNorm>(static_cast<int>(arg_int(a, "size", "rmsnorm")), static_cast<float>(arg_number(a, "eps", "rmsnorm")));
});
}  // namespace

}  // namespace vmb
