"""What every part has in common, and the two contexts a part sees: one when it is bound to its
weights, one for each step.

Interfaces (duck-typed; the classes below are conveniences, not requirements):

norm          weight_specs(); bind(w, bc); forward(ctx, h, delta, out, rows=None)
                h float32 [T, hid] residual; delta (activation dtype) is added to h first if given;
                out (activation dtype) receives norm(h) for all rows or for `rows`.
position      tables(bc) -> (inv_freq float32 tensor or None, rotary_dim)   [consumed by a mixer]
mixer         weight_specs(); bind(w, bc); cache_need() -> CacheNeed;
                forward(ctx, x, out): x, out [T, hid] activation dtype.  Reads/writes its cache through
                ctx.kv() / ctx.state(); knows sequences through ctx.positions, ctx.seq_of_token ...
feed_forward  weight_specs(); bind(w, bc); forward(ctx, x, out)
arrangement   built with (mixer, feed_forward, mixer_norm, feed_forward_norm); forward(ctx, h, pending)
                -> pending: wires norms, parts and the residual; `pending` is a delta not yet added to h.
embedding     weight_specs(); bind(w, bc); forward(ctx, tokens, h)
head          weight_specs(); bind(w, bc); forward(ctx, x_rows, logits)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from ..weights.loader import WeightSpec


@dataclass
class BindContext:
    """Where and in which dtype a model is being put on the device.  `uploads` de-duplicates host tensors that
    several parts share (a tied head and the embedding table), so they are one device tensor too."""
    dtype: torch.dtype
    device: torch.device
    uploads: Dict = field(default_factory=dict)

    def upload(self, t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        dtype = dtype or t.dtype
        key = (t.data_ptr(), tuple(t.shape), t.dtype, dtype)
        if key not in self.uploads:
            self.uploads[key] = t.to(device=self.device, dtype=dtype).contiguous()
        return self.uploads[key]

    def matrix_dtype(self, *stored: torch.Tensor) -> torch.dtype:
        """Dtype a weight matrix is kept in: the compute dtype, except that a tensor stored in 32-bit stays
        32-bit even when activations are bfloat16 (its products then run in float32)."""
        if self.dtype == torch.float32 or any(t.dtype == torch.float32 for t in stored):
            return torch.float32
        return self.dtype


class Part:
    # True only for parts whose `forward` launches the same work for every step of the same SHAPE (token,
    # sequence and row counts, table widths) and reads everything else from device memory: such a step can
    # be recorded into a CUDA graph.  A part that looks at host copies of the step (slots, lengths) says False.
    graph_safe = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def bind(self, weights: Dict[str, torch.Tensor], bc: BindContext) -> None:
        pass
