// Arrangements: how a layer wires its norms, mixer, feed-forward and the residual stream.
#include "args.h"
#include "../engine/ops.h"

namespace vmb {

// h += mixer(norm(h)); h += feed_forward(norm(h))  (examples/common/llama/llama_graph.cpp:203-229).
//
// The residual stream h is float32.  Each sum is carried out by the norm kernel that follows it, so `forward` takes the
// delta the previous layer left pending and returns its own last delta pending.  A part that can take the preceding norm
// into its first kernel and the residual sum into its last one (can_fuse / forward_fused) does so.
class PreNormBlock : public Arrangement {
public:
    explicit PreNormBlock(const BlockParts& p) : p_(p) {}
    bool graph_safe() const override { return true; }

    void* forward(StepContext& ctx, float* h, void* pending) override {
        const long long hid = hidden(ctx);
        if (p_.mixer->can_fuse(ctx, *p_.mixer_norm)) {
            settle(ctx, h, pending, hid);
            p_.mixer->forward_fused(ctx, h, *p_.mixer_norm);
            pending = nullptr;
        } else {
            void* x = ctx.take_tokens(hid, ctx.act_dtype);
            p_.mixer_norm->forward(ctx, h, pending, x, nullptr, 0);
            ctx.give(pending);
            pending = ctx.take_tokens(hid, ctx.act_dtype);
            p_.mixer->forward(ctx, x, pending);
            ctx.give(x);
        }
        if (p_.feed_forward->can_fuse(ctx, *p_.feed_forward_norm)) {
            settle(ctx, h, pending, hid);
            p_.feed_forward->forward_fused(ctx, h, *p_.feed_forward_norm);
            return nullptr;
        }
        void* x = ctx.take_tokens(hid, ctx.act_dtype);
        p_.feed_forward_norm->forward(ctx, h, pending, x, nullptr, 0);
        ctx.give(pending);
        void* out = ctx.take_tokens(hid, ctx.act_dtype);
        p_.feed_forward->forward(ctx, x, out);
        ctx.give(x);
        return out;
    }

private:
    static long long hidden(const StepContext& ctx) { return ctx.hidden; }
    // add a delta that is still pending to the residual stream
    static void settle(StepContext& ctx, float* h, void* pending, long long hid) {
        if (!pending) return;
        ops::residual_add(h, pending, static_cast<long long>(ctx.T) * hid, ctx.act_dtype, ctx.stream);
        ctx.give(pending);
    }
    BlockParts p_;
};

namespace {
struct Reg {
    Reg() {
        register_arrangement("prenorm", [](const json::Value&, const BlockParts& parts) { return std::make_shared<PreNormBlock>(parts); });
    }
} reg;
}  // namespace

}  // namespace vmb
