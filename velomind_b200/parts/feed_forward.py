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
        if getattr(norm, "as_rms", None) is None or ctx.act_dtype != torch.bfloat16:
            return False
        if self.gate_up.weight.dtype != torch.bfloat16 or self.down.weight.dtype != torch.bfloat16:
            return False
        if ctx.T <= ops.SKINNY_MAX_ROWS:
            return self.hidden % 32 == 0 and self.intermediate % 32 == 0
        return ops.tc_fused_rows(ctx.T) and self.hidden % 8 == 0 and self.intermediate % 64 == 0

    def forward_fused(self, ctx, h: torch.Tensor, norm) -> None:
        """h += down(silu(gate(norm(h))) * up(norm(h))): two or three launches."""
        act = ctx.take_tokens(self.intermediate, torch.bfloat16)
        skinny = ctx.T <= ops.SKINNY_MAX_ROWS
        if skinny and ctx.T <= ops.SKINNY_NORM_ROWS:
            ops.skinny_swiglu(h, norm.as_rms(), self.gate_up.weight, act)
        else:
            x = ctx.take_tokens(self.hidden, torch.bfloat16)          # many rows: norm once, not once per CTA
            norm.forward(ctx, h, None, x)
            if skinny:
                ops.skinny_swiglu(x, None, self.gate_up.weight, act)
            else:
                ops.tc_swiglu(x, self.gate_up.weight, act, ctx.err)
            ctx.ws.give(x)
        if skinny:
            ops.skinny_linear(act, None, self.down.weight, None, residual=h)
        else:
            ops.tc_linear(act, self.down.weight, None, residual=h, err=ctx.err)
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
