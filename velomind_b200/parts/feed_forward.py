"""Gated feed-forward (SwiGLU)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import BindContext, Part
from .linear import Linear
from .registry import register_part


class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)), no biases (examples/common/llama/llama_graph.cpp:22-28,122-138).
    gate and up are one stacked product; the activation kernel reads both halves."""

    graph_safe = True

    def __init__(self, hidden: int, intermediate: int):
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.gate_up = self.down = None

    def weight_specs(self):
        return {
            "gate_proj.weight": WeightSpec((self.intermediate, self.hidden)),
            "up_proj.weight": WeightSpec((self.intermediate, self.hidden)),
            "down_proj.weight": WeightSpec((self.hidden, self.intermediate)),
        }

    def bind(self, weights, bc: BindContext) -> None:
        self.gate_up = Linear([weights["gate_proj.weight"], weights["up_proj.weight"]], bc)
        self.down = Linear([weights["down_proj.weight"]], bc)

    def can_fuse(self, ctx, norm) -> bool:
        rms = getattr(norm, "as_rms", None)
        return (rms is not None and ctx.act_dtype == torch.bfloat16 and ops.skinny_ok(ctx.T, self.hidden, self.gate_up.weight)
                and ops.skinny_ok(ctx.T, self.intermediate, self.down.weight) and self.intermediate % 8 == 0
                and self.hidden % 8 == 0)

    def forward_fused(self, ctx, h: torch.Tensor, norm) -> None:
        """h += down(silu(gate(norm(h))) * up(norm(h))) in two launches (few tokens, bfloat16)."""
        x, rms = h, norm.as_rms()
        if ctx.T > ops.SKINNY_NORM_ROWS:          # many rows: norm once, not once per CTA
            x, rms = ctx.take_tokens(self.hidden, torch.bfloat16), None
            norm.forward(ctx, h, None, x)
        act = ctx.take_tokens(self.intermediate, torch.bfloat16)
        ops.skinny_swiglu(x, rms, self.gate_up.weight, act)
        if x is not h:
            ctx.ws.give(x)
        ops.skinny_linear(act, None, self.down.weight, None, residual=h)
        ctx.ws.give(act)

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor) -> None:
        gu = ctx.take_tokens(2 * self.intermediate, x.dtype)
        self.gate_up(ctx, x, gu)
        act = ctx.take_tokens(self.intermediate, x.dtype)
        ops.swiglu(gu, act)
        ctx.ws.give(gu)
        self.down(ctx, act, out)
        ctx.ws.give(act)


register_part("feed_forward", "swiglu", SwiGLU)
