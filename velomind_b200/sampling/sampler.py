"""Sampling parameters and the device sampler.

Option names and defaults follow the reference's command line
(examples/smollm2/interactive_main.cpp:23-25,39-41): `--temp` 0.7 (0 or less:
greedy), `--top-p` 0.9 (0 or less: greedy), `--max-tokens` 32; its fixed seed is
42 (:113).  The rule itself is in csrc/sampling.cu.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops


def _host_buffer(shape, dtype: torch.dtype) -> torch.Tensor:
    return torch.empty(shape, dtype=dtype, pin_memory=True)


def _sync() -> None:
    torch.cuda.current_stream().synchronize()


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_p: float = 0.9
    max_tokens: int = 32
    seed: int = 42
    stop_tokens: Tuple[int, ...] = ()

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0 or self.top_p <= 0


class DeviceSampler:
    """Draws one token per row of logits on the device.  A row's draw depends on (seed, stream, step) of
    its request only, never on the rest of the batch."""

    FIELDS = 5   # temperature, top_p (float32 bit patterns in an int64 lane), seed, stream, step

    def __init__(self, device, max_rows: int = 64):
        self.device = torch.device(device)
        self._alloc(max_rows)

    def _alloc(self, rows: int) -> None:
        self.rows = rows
        # one byte buffer: int64 seed, stream, step [3, rows], then float32 temperature, top_p [2, rows]: ONE host-to-device copy
        nbytes = 3 * 8 * rows + 2 * 4 * rows
        self.host = _host_buffer((nbytes,), torch.uint8)
        self.dev = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        split = 3 * 8 * rows
        self.host_i = self.host[:split].view(torch.int64).view(3, rows)
        self.host_f = self.host[split:].view(torch.float32).view(2, rows)
        self.dev_i = self.dev[:split].view(torch.int64).view(3, rows)
        self.dev_f = self.dev[split:].view(torch.float32).view(2, rows)
        self.out = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.out_host = _host_buffer((rows,), torch.int32)
        # where the kernel can write into pinned host memory itself, no copy follows it
        self.out_direct = ops.host_device_pointer(self.out_host) if self.device.type == "cuda" else 0
        self._uploaded = None          # (params, streams, steps) that the device's parameter block holds

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], streams: Sequence[int],
               steps: Sequence[int]) -> np.ndarray:
        """Tokens (host int32 array) for logits [R, V]; row r uses params[r] and the Philox counter
        (steps[r], streams[r])."""
        R = logits.shape[0]
        if R == 0:
            return np.zeros(0, dtype=np.int32)
        if R > self.rows:
            self._alloc(max(R, 2 * self.rows))
        params, streams, steps = list(params), list(streams), list(steps)
        step_add = None
        up = self._uploaded
        if up is not None and up[0] == params and up[1] == streams:
            # the same requests as at the last upload: if all of them have moved on by the same number of draws,
            # the block on the device still serves, and that number goes to the kernel as an argument
            step_add = steps[0] - up[2][0]
            if any(s - b != step_add for s, b in zip(steps, up[2])):
                step_add = None
        if step_add is None:
            hf, hi = self.host_f.numpy(), self.host_i.numpy()
            for r, p in enumerate(params):
                hf[0, r], hf[1, r] = p.temperature, p.top_p
                hi[0, r], hi[1, r], hi[2, r] = p.seed, streams[r], steps[r]
            self.dev.copy_(self.host, non_blocking=True)
            ops.h2d_bytes += self.host.numel()
            self._uploaded = (params, streams, steps)
            step_add = 0
        args = (logits, self.dev_f[0, :R], self.dev_f[1, :R], self.dev_i[0, :R], self.dev_i[1, :R], self.dev_i[2, :R])
        if self.out_direct:
            ops.sample(*args, self.out_direct, step_add)
        else:
            ops.sample(*args, self.out, step_add)
            self.out_host.copy_(self.out, non_blocking=True)
        _sync()
        ops.d2h_bytes += 4 * R
        return self.out_host.numpy()[:R].copy()
