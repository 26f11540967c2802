"""A bias-free linear map y = x W^T with W in the checkpoint's [out, in] layout.

Several checkpoint matrices that read the same input can be stacked into one
(q/k/v, gate/up): one product instead of three.  The reference transposes each
matrix to [in, out] and multiplies one by one (examples/smollm2/model_loader.cpp:176-233,
examples/common/llama/llama_graph.cpp:63-65); [out, in] rows are K-contiguous,
which is what the tensor-core and weight-streaming kernels want.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops
from .base import BindContext


class Linear:
    def __init__(self, stored: Sequence[torch.Tensor], bc: BindContext):
        dtype = bc.matrix_dtype(*stored)
        if len(stored) == 1:
            self.weight = bc.upload(stored[0], dtype)
        else:
            self.weight = torch.cat([t.to(dtype) for t in stored], dim=0).to(bc.device).contiguous()
        self.out_features, self.in_features = self.weight.shape

    def __call__(self, ctx, x: torch.Tensor, out: torch.Tensor) -> None:
        """out = x W^T.  out may be float32 under bfloat16 inputs (logits)."""
        if x.dtype == self.weight.dtype:
            if out.dtype == x.dtype or out.dtype == torch.float32:
                ops.linear(x, self.weight, out)
                return
        elif self.weight.dtype != torch.float32:
            raise ops.KernelError(f"linear: input {x.dtype} does not fit weights kept in {self.weight.dtype}")
        # 32-bit weights under bfloat16 activations: widen the input, multiply in float32, narrow the result
        x32 = x
        if x.dtype != torch.float32:
            x32 = ctx.ws.take(x.shape, torch.float32)
            ops.convert(x, x32)
        if out.dtype == torch.float32:
            ops.linear(x32, self.weight, out)
        else:
            y32 = ctx.ws.take(out.shape, torch.float32)
            ops.linear(x32, self.weight, y32)
            ops.convert(y32, out)
            ctx.ws.give(y32)
        if x32 is not x:
            ctx.ws.give(x32)
