"""Token embedding table and the output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import BindContext, Part
from .linear import Linear
from .registry import register_part


class TokenEmbedding(Part):
    """h[t, :] = table[token[t], :] into the float32 residual stream (src/cpu/ops/embedding.cpp:27-32)."""

    graph_safe = True

    def __init__(self, vocab: int, hidden: int):
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.table = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab, self.hidden))}

    def bind(self, weights, bc: BindContext) -> None:
        self.table = bc.upload(weights["weight"], bc.matrix_dtype(weights["weight"]))

    def forward(self, ctx, tokens, h) -> None:
        ops.embed_gather(self.table, tokens, h, ctx.err)


class LinearHead(Part):
    """logits = x W^T in float32.  `tied_to` names the tensor that stands in when the checkpoint has no
    head of its own (examples/smollm2/model_loader.cpp:124-158: lm_head.weight if present, else the
    embedding when tied); the device tensor is then shared with the embedding, not copied."""

    graph_safe = True

    def __init__(self, vocab: int, hidden: int, tied_to: str | None = None):
        self.vocab, self.hidden, self.tied_to = int(vocab), int(hidden), tied_to
        self.proj = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.vocab, self.hidden), alias_of=self.tied_to)}

    def bind(self, weights, bc: BindContext) -> None:
        self.proj = Linear([weights["weight"]], bc)

    def forward(self, ctx, x, logits) -> None:
        w = self.proj.weight
        if x.dtype == torch.bfloat16 and ops.skinny_ok(x.shape[0], self.hidden, w) and self.vocab % 8 == 0:
            ops.skinny_linear(x, None, w, logits)        # few rows: stream the table once, float32 logits
        else:
            self.proj(ctx, x, logits)


register_part("embedding", "token_table", TokenEmbedding)
register_part("head", "linear", LinearHead)
