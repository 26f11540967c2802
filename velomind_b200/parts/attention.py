"""Grouped-query attention over the cache, as a mixer."""
from __future__ import annotations

import math

import torch

from ..cache.store import CacheNeed
from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import BindContext, Part
from .linear import Linear
from .registry import build_part, register_part
from .spec import PartSpec


class GroupedQueryAttention(Part):
    """q, k, v projections (one stacked product), position encoding of q and k fused with the cache write,
    causal attention of each new token over its sequence's cache, output projection.

    Reference: examples/common/llama/llama_graph.cpp:53-120 (projections, head split, rotary, scores,
    softmax, context, output projection) and :217-222 (query head h reads kv head h / G).  The reference
    folds 1/sqrt(head_dim) into Wq when it loads real weights (examples/smollm2/model_loader.cpp:277);
    here `scale` multiplies the query inside the attention kernel, which is the same number.

    `window` > 0 limits a query to the last `window` keys (itself included); 0 means all earlier keys.
    """

    graph_safe = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, position: PartSpec,
                 window: int = 0, scale: float | None = None):
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", position)
        self.qkv = self.out = None
        self.inv_freq, self.rotary_dim = None, 0

    def weight_specs(self):
        H, Hkv, D, hid = self.heads, self.kv_heads, self.head_dim, self.hidden
        return {
            "q_proj.weight": WeightSpec((H * D, hid)),
            "k_proj.weight": WeightSpec((Hkv * D, hid)),
            "v_proj.weight": WeightSpec((Hkv * D, hid)),
            "o_proj.weight": WeightSpec((hid, H * D)),
        }

    def bind(self, weights, bc: BindContext) -> None:
        self.qkv = Linear([weights["q_proj.weight"], weights["k_proj.weight"], weights["v_proj.weight"]], bc)
        self.out = Linear([weights["o_proj.weight"]], bc)
        self.inv_freq, self.rotary_dim = self.position.tables(bc)

    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window > 0 else "all", self.kv_heads, self.head_dim, self.window)

    def can_fuse(self, ctx, norm) -> bool:
        """True if this step can run as: [norm +] qkv + rotary + cache write -> attention -> out + residual,
        with the weight-streaming kernels (few tokens) or the tensor-core kernels (many tokens)."""
        if getattr(norm, "as_rms", None) is None or ctx.act_dtype != torch.bfloat16:
            return False
        if self.qkv.weight.dtype != torch.bfloat16 or self.out.weight.dtype != torch.bfloat16:
            return False
        if self.rotary_dim not in (0, self.head_dim) or self.hidden % 8 or (self.heads * self.head_dim) % 8:
            return False
        if ctx.T <= ops.SKINNY_MAX_ROWS:
            return self.hidden % 32 == 0 and (self.heads * self.head_dim) % 32 == 0 and self.head_dim % 16 == 0
        return ops.tc_fused_rows(ctx.T) and self.head_dim in (64, 128)

    def forward_fused(self, ctx, h: torch.Tensor, norm) -> None:
        """h += attention(norm(h)): three or four launches."""
        H, Hkv, D = self.heads, self.kv_heads, self.head_dim
        q = ctx.take_tokens(H * D, torch.bfloat16)
        k_pages, v_pages, table, owns = ctx.kv()
        kp, vp = (k_pages, v_pages) if owns else (None, None)
        skinny = ctx.T <= ops.SKINNY_MAX_ROWS
        if skinny and ctx.T <= ops.SKINNY_NORM_ROWS:
            ops.skinny_qkv_rope(h, norm.as_rms(), self.qkv.weight, q, ctx.positions, ctx.seq_of_token, table, self.inv_freq,
                                self.rotary_dim, kp, vp, H, Hkv, D, ctx.err)
        else:
            x = ctx.take_tokens(self.hidden, torch.bfloat16)          # many rows: norm once, not once per CTA
            norm.forward(ctx, h, None, x)
            qkv_rope = ops.skinny_qkv_rope if skinny else ops.tc_qkv_rope
            args = (x, None, self.qkv.weight) if skinny else (x, self.qkv.weight)
            qkv_rope(*args, q, ctx.positions, ctx.seq_of_token, table, self.inv_freq, self.rotary_dim, kp, vp, H, Hkv, D, ctx.err)
            ctx.ws.give(x)
        att = ctx.take_tokens(H * D, torch.bfloat16)
        ops.attention(ctx, q, H * D, k_pages, v_pages, table, att, H, Hkv, D, self.scale, self.window)
        ctx.ws.give(q)
        if skinny:
            ops.skinny_linear(att, None, self.out.weight, None, residual=h)
        else:
            ops.tc_linear(att, self.out.weight, None, residual=h, err=ctx.err)
        ctx.ws.give(att)

    def forward(self, ctx, x: torch.Tensor, out: torch.Tensor) -> None:
        H, Hkv, D = self.heads, self.kv_heads, self.head_dim
        width = (H + 2 * Hkv) * D
        qkv = ctx.take_tokens(width, x.dtype)
        self.qkv(ctx, x, qkv)
        k_pages, v_pages, table, owns = ctx.kv()
        ops.rope_kv_write(qkv, ctx.positions, ctx.seq_of_token, table, self.inv_freq, self.rotary_dim,
                          k_pages if owns else None, v_pages if owns else None, H, Hkv, D, ctx.err)
        att = ctx.take_tokens(H * D, x.dtype)
        ops.attention(ctx, qkv, width, k_pages, v_pages, table, att, H, Hkv, D, self.scale, self.window)
        ctx.ws.give(qkv)
        self.out(ctx, att, out)
        ctx.ws.give(att)


register_part("mixer", "grouped_query_attention", GroupedQueryAttention)
