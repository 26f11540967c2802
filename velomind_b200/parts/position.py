"""Position encodings.  A position part owns constants only; the mixer's kernels apply them."""
from __future__ import annotations

import numpy as np
import torch

from .base import BindContext, Part
from .registry import register_part


class RotaryHalfSplit(Part):
    """Rotary positions on half-split pairs (j, j + rotary_dim/2).  Frequencies as the reference builds
    them, in float32: inv_freq[j] = 1 / pow(theta, 2j / rotary_dim)
    (examples/common/llama/llama_rope_mask.cpp:17-19); the angle pos * inv_freq[j] and its sine and cosine
    are computed in float32 on the device."""

    graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim) if rotary_dim is not None else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within the head size {self.head_dim}")
        self.theta = float(theta)
        self._inv_freq = None

    def inv_freq_host(self) -> np.ndarray:
        j = np.arange(self.rotary_dim // 2, dtype=np.float32)
        exponent = (np.float32(2) * j) / np.float32(self.rotary_dim)
        return (np.float32(1.0) / np.power(np.float32(self.theta), exponent, dtype=np.float32)).astype(np.float32)

    def tables(self, bc: BindContext):
        if self._inv_freq is None:
            self._inv_freq = torch.from_numpy(self.inv_freq_host()).to(bc.device)
        return self._inv_freq, self.rotary_dim


class NoPosition(Part):
    """No position encoding: queries and keys pass unrotated."""

    graph_safe = True

    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def tables(self, bc: BindContext):
        return None, 0


register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "none", NoPosition)
