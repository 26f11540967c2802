"""Arrangements: how a layer wires its norms, mixer, feed-forward and the residual stream."""
from __future__ import annotations

from ..kernels import ops
from .registry import register_part


class PreNormBlock:
    """h += mixer(norm(h)); h += feed_forward(norm(h))  (examples/common/llama/llama_graph.cpp:203-229).

    The residual stream h is float32.  Each sum is carried out by the norm kernel that follows it, so
    `forward` takes the delta the previous layer left pending and returns its own last delta pending.
    """

    graph_safe = True

    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self):
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, ctx, h, pending):
        hid = h.shape[1]
        # A part that can take the preceding norm into its first kernel and the residual sum into its last one
        # (`can_fuse` / `forward_fused`) does so; otherwise norm, part and sum are separate steps, the sum being
        # carried out by the next norm kernel.
        if getattr(self.mixer, "can_fuse", None) is not None and self.mixer.can_fuse(ctx, self.mixer_norm):
            self._settle(ctx, h, pending)
            self.mixer.forward_fused(ctx, h, self.mixer_norm)
            pending = None
        else:
            x = ctx.take_tokens(hid, ctx.act_dtype)
            self.mixer_norm.forward(ctx, h, pending, x)
            ctx.ws.give(pending)
            pending = ctx.take_tokens(hid, ctx.act_dtype)
            self.mixer.forward(ctx, x, pending)
            ctx.ws.give(x)
        if getattr(self.feed_forward, "can_fuse", None) is not None and self.feed_forward.can_fuse(ctx, self.feed_forward_norm):
            self._settle(ctx, h, pending)
            self.feed_forward.forward_fused(ctx, h, self.feed_forward_norm)
            return None
        x = ctx.take_tokens(hid, ctx.act_dtype)
        self.feed_forward_norm.forward(ctx, h, pending, x)
        ctx.ws.give(pending)
        out = ctx.take_tokens(hid, ctx.act_dtype)
        self.feed_forward.forward(ctx, x, out)
        ctx.ws.give(x)
        return out

    @staticmethod
    def _settle(ctx, h, pending) -> None:
        """Add a delta that is still pending to the residual stream."""
        if pending is not None:
            ops.residual_add(h, pending)
            ctx.ws.give(pending)


register_part("arrangement", "prenorm", PreNormBlock)
