"""Root-mean-square norm with a learned scale."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import BindContext, Part
from .registry import register_part


class RMSNorm(Part):
    """y = x / sqrt(mean(x^2) + eps) * weight, statistics in float32 (src/cpu/ops/rmsnorm.cpp:42-59).
    The residual add that precedes a norm in a pre-norm block is fused into the same kernel."""

    graph_safe = True

    def __init__(self, size: int, eps: float):
        self.size = int(size)
        self.eps = float(eps)
        self.weight = None

    def weight_specs(self):
        return {"weight": WeightSpec((self.size,), "float", "ones")}

    def bind(self, weights, bc: BindContext) -> None:
        self.weight = bc.upload(weights["weight"], torch.float32)   # exact for BF16 and F32 storage

    def as_rms(self):
        """(weight, eps) for kernels that fuse this norm into the product that follows it."""
        return self.weight, self.eps

    def forward(self, ctx, h, delta, out, rows=None) -> None:
        ops.add_rmsnorm(h, delta, self.weight, self.eps, out, rows)


register_part("norm", "rmsnorm", RMSNorm)
