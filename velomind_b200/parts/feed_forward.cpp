// Gated feed-forward (SwiGLU).
#include "args.h"
#include "linear.h"

namespace vmb {

// down(silu(gate(x)) * up(x)), no biases (examples/common/llama/llama_graph.cpp:22-28,122-138).  gate and up are one
// stacked product; the activation kernel reads both halves.
class SwiGLU : public FeedForward {
public:
    SwiGLU(int hidden, int intermediate) : hidden_(hidden), I_(intermediate) {}

    WeightTable weight_specs() const override {
        WeightTable t;
        t["gate_proj.weight"].shape = {I_, hidden_};
        t["up_proj.weight"].shape = {I_, hidden_};
        t["down_proj.weight"].shape = {hidden_, I_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        gate_up_.bind({&w.at("gate_proj.weight"), &w.at("up_proj.weight")}, bc);
        down_.bind({&w.at("down_proj.weight")}, bc);
    }

    bool graph_safe() const override { return true; }

    // rows up to which the weight-streaming kernels take this part (fewer when its matrices are large)
    int max_rows() const {
        return ops::skinny_max_rows(2 * std::max(gate_up_.weight.rows() * gate_up_.weight.cols(), down_.weight.rows() * down_.weight.cols()));
    }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (gate_up_.weight.dtype != DType::BF16 || down_.weight.dtype != DType::BF16) return false;
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && I_ % 32 == 0;
        return hidden_ % 8 == 0 && I_ % 8 == 0;
    }

    // h += down(silu(gate(norm(h))) * up(norm(h))): two or three launches.
    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const bool skinny = ctx.T_cap <= max_rows();
        const bool tc = !skinny && ops::tc_fused_rows(ctx) && I_ % 64 == 0;
        if (!skinny && !tc) {
            // the library's products: norm, gate and up, SwiGLU, down added into h by the product itself
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            void* gu = ctx.take_tokens(2ll * I_, DType::BF16);
            ops::linear(x, DType::BF16, hidden_, gate_up_.weight, gu, DType::BF16, ctx.T, ctx.stream);
            ctx.give(x);
            void* a = ctx.take_tokens(I_, DType::BF16);
            ops::swiglu(gu, a, ctx.T, I_, DType::BF16, ctx.stream);
            ctx.give(gu);
            ops::linear_residual(a, I_, down_.weight, h, ctx.T, ctx.stream);
            ctx.give(a);
            return;
        }
        void* act = ctx.take_tokens(I_, DType::BF16);
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_swiglu(h, nw, eps, gate_up_.weight, ctx.T, I_, act, ctx.err, ctx.stream);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);           // many rows: norm once, not once per CTA
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) ops::skinny_swiglu(x, nullptr, 0.f, gate_up_.weight, ctx.T, I_, act, ctx.err, ctx.stream);
            else ops::tc_swiglu(x, hidden_, gate_up_.weight, ctx.T, I_, act, ctx.err, ctx.stream);
            ctx.give(x);
        }
        if (skinny) ops::skinny_linear(act, nullptr, 0.f, down_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::tc_linear(act, I_, down_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(act);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        void* gu = ctx.take_tokens(2ll * I_, ctx.act_dtype);
        gate_up_.apply(ctx, x, ctx.act_dtype, gu, ctx.act_dtype, ctx.T, ctx.T_cap);
        void* act = ctx.take_tokens(I_, ctx.act_dtype);
        ops::swiglu(gu, act, ctx.T, I_, ctx.act_dtype, ctx.stream);
        ctx.give(gu);
        down_.apply(ctx, act, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(act);
    }

private:
    int hidden_, I_;
    Linear gate_up_, down_;
};

namespace {
RegisterPart reg("feed_forward", "swiglu", [](const json::Value& a) {
    return std::make_shared<SwiGLU>(static_cast<int>(arg_int(a, "hidden", "swiglu")), static_cast<int>(arg_int(a, "intermediate", "swiglu")));
});
}  // namespace

}  // namespace vmb
