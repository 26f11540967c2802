// Grouped-query attention over the cache, as a mixer.
#include <cmath>

#include "args.h"
#include "linear.h"

namespace vmb {

// q, k, v projections (one stacked product), position encoding of q and k fused with the cache write, causal attention of
// each new token over its sequence's cache, output projection.
//
// Reference: examples/common/llama/llama_graph.cpp:53-120 (projections, head split, rotary, scores, softmax, context,
// output projection) and :217-222 (query head h reads kv head h / G).  The reference folds 1/sqrt(head_dim) into Wq when it
// loads real weights (examples/smollm2/model_loader.cpp:277); here `scale` multiplies the query inside the attention
// kernel, which is the same number.
//
// `window` > 0 limits a query to the last `window` keys (itself included); 0 means all earlier keys.
class GroupedQueryAttention : public Mixer {
public:
    GroupedQueryAttention(int hidden, int heads, int kv_heads, int head_dim, const PartSpec& position, int window, double scale)
        : hidden_(hidden), H_(heads), Hkv_(kv_heads), D_(head_dim), window_(window),
          scale_(scale > 0 ? static_cast<float>(scale) : static_cast<float>(1.0 / std::sqrt(static_cast<double>(head_dim)))),
          position_(build_part_as<Position>("position", position)) {
        if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) throw ConfigError(format("heads (%d) must be a multiple of kv_heads (%d)", heads, kv_heads));
    }

    WeightTable weight_specs() const override {
        WeightTable t;
        t["q_proj.weight"].shape = {static_cast<long long>(H_) * D_, hidden_};
        t["k_proj.weight"].shape = {static_cast<long long>(Hkv_) * D_, hidden_};
        t["v_proj.weight"].shape = {static_cast<long long>(Hkv_) * D_, hidden_};
        t["o_proj.weight"].shape = {hidden_, static_cast<long long>(H_) * D_};
        return t;
    }

    void bind(const Weights& w, BindContext& bc) override {
        qkv_.bind({&w.at("q_proj.weight"), &w.at("k_proj.weight"), &w.at("v_proj.weight")}, bc);
        out_.bind({&w.at("o_proj.weight")}, bc);
        rotary_ = position_->tables(bc);
    }

    bool graph_safe() const override { return position_->graph_safe(); }

    CacheNeed cache_need() const override {
        CacheNeed n;
        n.kind = window_ > 0 ? CacheNeed::Window : CacheNeed::All;
        n.kv_heads = Hkv_;
        n.key_dim = n.value_dim = D_;
        n.window = window_;
        return n;
    }

    // True if this step can run as: [norm +] qkv + rotary + cache write -> attention -> out + residual, with the
    // weight-streaming kernels (few tokens), the tensor-core kernels (many tokens, when asked for) or the library products
    // (the out projection then adds into the residual stream as its own accumulator).
    // rows up to which the weight-streaming kernels take this part (fewer when its matrices are large)
    int max_rows() const {
        return ops::skinny_max_rows(2 * std::max(qkv_.weight.rows() * qkv_.weight.cols(), out_.weight.rows() * out_.weight.cols()));
    }

    bool can_fuse(const StepContext& ctx, const Norm& norm) const override {
        const float* nw;
        float eps;
        if (!norm.as_rms(&nw, &eps) || ctx.act_dtype != DType::BF16) return false;
        if (qkv_.weight.dtype != DType::BF16 || out_.weight.dtype != DType::BF16) return false;
        if (hidden_ % 8 || (H_ * D_) % 8) return false;
        const bool fused_rotary = rotary_.rotary_dim == 0 || (rotary_.rotary_dim == D_ && rotary_.pairing == VM_PAIR_HALF_SPLIT);
        if (!fused_rotary) return ctx.T_cap > max_rows();      // (the library path rotates with the kernel of its own)
        if (ctx.T_cap <= max_rows()) return hidden_ % 32 == 0 && (H_ * D_) % 32 == 0 && D_ % 16 == 0;
        return true;
    }

    // h += attention(norm(h)): three or four launches, five on the library path.
    void forward_fused(StepContext& ctx, float* h, Norm& norm) override {
        const float* nw = nullptr;
        float eps = 0.f;
        norm.as_rms(&nw, &eps);
        const KVView kv = ctx.kv();
        const bool skinny = ctx.T_cap <= max_rows();
        const bool fused_rotary = rotary_.rotary_dim == 0 || (rotary_.rotary_dim == D_ && rotary_.pairing == VM_PAIR_HALF_SPLIT);
        const bool tc = !skinny && fused_rotary && ops::tc_fused_rows(ctx) && (D_ == 64 || D_ == 128);
        if (!skinny && !tc) {
            // the library's products: norm, q k v, rotary + cache write, attention, out added into h by the product itself
            const long long width = static_cast<long long>(H_ + 2 * Hkv_) * D_;
            void* x = ctx.take_tokens(hidden_, DType::BF16);
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            void* qkv = ctx.take_tokens(width, DType::BF16);
            ops::linear(x, DType::BF16, hidden_, qkv_.weight, qkv, DType::BF16, ctx.T, ctx.stream);
            ctx.give(x);
            ops::rope_kv_write(qkv, ctx, kv, rotary_, H_, Hkv_, D_, DType::BF16);
            void* att = ctx.take_tokens(static_cast<long long>(H_) * D_, DType::BF16);
            ops::attention(ctx, qkv, static_cast<int>(width), kv, att, H_, Hkv_, D_, scale_, window_);
            ctx.give(qkv);
            ops::linear_residual(att, static_cast<long long>(H_) * D_, out_.weight, h, ctx.T, ctx.stream);
            ctx.give(att);
            return;
        }
        void* q = ctx.take_tokens(static_cast<long long>(H_) * D_, DType::BF16);
        if (skinny && ctx.T_cap <= ops::SKINNY_NORM_ROWS) {
            ops::skinny_qkv_rope(h, nw, eps, qkv_.weight, q, ctx, kv, rotary_, H_, Hkv_, D_);
        } else {
            void* x = ctx.take_tokens(hidden_, DType::BF16);           // many rows: norm once, not once per CTA
            norm.forward(ctx, h, nullptr, x, nullptr, 0);
            if (skinny) ops::skinny_qkv_rope(x, nullptr, 0.f, qkv_.weight, q, ctx, kv, rotary_, H_, Hkv_, D_);
            else ops::tc_qkv_rope(x, hidden_, qkv_.weight, q, ctx, kv, rotary_, H_, Hkv_, D_);
            ctx.give(x);
        }
        void* att = ctx.take_tokens(static_cast<long long>(H_) * D_, DType::BF16);
        ops::attention(ctx, q, H_ * D_, kv, att, H_, Hkv_, D_, scale_, window_);
        ctx.give(q);
        if (skinny) ops::skinny_linear(att, nullptr, 0.f, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        else ops::tc_linear(att, static_cast<long long>(H_) * D_, out_.weight, ctx.T, nullptr, hidden_, false, h, ctx.err, ctx.stream);
        ctx.give(att);
    }

    void forward(StepContext& ctx, const void* x, void* out) override {
        const long long width = static_cast<long long>(H_ + 2 * Hkv_) * D_;
        void* qkv = ctx.take_tokens(width, ctx.act_dtype);
        qkv_.apply(ctx, x, ctx.act_dtype, qkv, ctx.act_dtype, ctx.T, ctx.T_cap);
        const KVView kv = ctx.kv();
        ops::rope_kv_write(qkv, ctx, kv, rotary_, H_, Hkv_, D_, ctx.act_dtype);
        void* att = ctx.take_tokens(static_cast<long long>(H_) * D_, ctx.act_dtype);
        ops::attention(ctx, qkv, static_cast<int>(width), kv, att, H_, Hkv_, D_, scale_, window_);
        ctx.give(qkv);
        out_.apply(ctx, att, ctx.act_dtype, out, ctx.act_dtype, ctx.T, ctx.T_cap);
        ctx.give(att);
    }

private:
    int hidden_, H_, Hkv_, D_, window_;
    float scale_;
    std::shared_ptr<Position> position_;
    Linear qkv_, out_;
    RotaryTable rotary_;
};

namespace {
RegisterPart reg("mixer", "grouped_query_attention", [](const json::Value& a) {
    const char* k = "grouped_query_attention";
    const json::Value* pos = a.find("position");
    if (!pos) throw ConfigError("part 'grouped_query_attention': argument 'position' (a part) is missing");
    return std::make_shared<GroupedQueryAttention>(static_cast<int>(arg_int(a, "hidden", k)), static_cast<int>(arg_int(a, "heads", k)),
                                                   static_cast<int>(arg_int(a, "kv_heads", k)), static_cast<int>(arg_int(a, "head_dim", k)),
                                                   part_spec_from_json(*pos, "grouped_query_attention.position"),
                                                   static_cast<int>(arg_int_or(a, "window", 0, k)), arg_number_or(a, "scale", 0.0, k));
});
}  // namespace

}  // namespace vmb
