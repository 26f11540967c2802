// Token embedding table and the output head.
#include "args.h"
#include "linear.h"

namespace vmb {

// h[t, :] = table[token[t], :] into the float32 residual stream (src/cpu/ops/embedding.cpp:27-32).
class TokenEmbedding : public Embedding {
public:
    TokenEmbedding(int vocab, int hidden) : vocab_(vocab), hidden_(hidden) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t["weight"].shape = {vocab_, hidden_};
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override { table_ = bc.upload(w.at("weight"), bc.matrix_dtype({&w.at("weight")})); }
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const int* tokens, float* h) override { ops::embed_gather(table_, tokens, h, ctx.T, hidden_, ctx.err, ctx.stream); }

private:
    int vocab_, hidden_;
    DeviceTensor table_;
};

// logits = x W^T in float32.  `tied_to` names the tensor that stands in when the checkpoint has no head of its own
// (examples/smollm2/model_loader.cpp:124-158: lm_head.weight if present, else the embedding when tied); the device tensor is
// then shared with the embedding, not copied.
class LinearHead : public Head {
public:
    LinearHead(int vocab, int hidden, std::string tied_to) : vocab_(vocab), hidden_(hidden), tied_to_(std::move(tied_to)) {}
    WeightTable weight_specs() const override {
        WeightTable t;
        t["weight"].shape = {vocab_, hidden_};
        t["weight"].alias_of = tied_to_;
        return t;
    }
    void bind(const Weights& w, BindContext& bc) override { proj_.bind({&w.at("weight")}, bc); }
    bool graph_safe() const override { return true; }
    void forward(StepContext& ctx, const void* x, float* logits) override {
        if (ctx.act_dtype == DType::BF16 && ops::skinny_ok(ctx.R, hidden_, proj_.weight) && vocab_ % 8 == 0 && ctx.R_cap <= ops::SKINNY_HEAD_MAX_ROWS)
            ops::skinny_linear(x, nullptr, 0.f, proj_.weight, ctx.R, logits, vocab_, true, nullptr, ctx.err, ctx.stream);   // few rows: stream the table once
        else
            proj_.apply(ctx, x, ctx.act_dtype, logits, DType::F32, ctx.R, ctx.R_cap);
    }

private:
    int vocab_, hidden_;
    std::string tied_to_;
    Linear proj_;
};

namespace {
RegisterPart reg_embed("embedding", "token_table", [](const json::Value& a) {
    return std::make_shared<TokenEmbedding>(static_cast<int>(arg_int(a, "vocab", "token_table")), static_cast<int>(arg_int(a, "hidden", "token_table")));
});
RegisterPart reg_head("head", "linear", [](const json::Value& a) {
    return std::make_shared<LinearHead>(static_cast<int>(arg_int(a, "vocab", "linear")), static_cast<int>(arg_int(a, "hidden", "linear")),
                                        arg_string_or(a, "tied_to", "", "linear"));
});
}  // namespace

}  // namespace vmb
