"""Activation memory of a step: liveness intervals packed into one arena, planned once per capacity.

The reference plans every graph build: liveness over the topological order,
then best-fit-decreasing placement into one arena with 256-byte alignment
(src/internal/graph_compiler.cpp:147-191 liveness, :286-398 placement, sort
by size, then lifetime, then birth; candidate offsets are 0 and the ends of
placed buffers that are alive at the same time), and reports peak bytes,
buffers, reuse and bytes saved (include/velomind/graph.h:40-46).

Here the parts ask for and give back buffers while a step runs.  The first
step of a capacity bucket records that sequence (with ordinary allocations);
the plan made from it serves every later step of the bucket from one arena,
with no allocation.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

ALIGN = 256


def _align(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


@dataclass(frozen=True)
class ArenaPlan:
    offsets: Tuple[int, ...]
    sizes: Tuple[int, ...]
    peak_bytes: int
    buffer_count: int
    reused_count: int           # buffers placed over bytes an earlier (dead) buffer used
    bytes_saved: int            # sum of sizes - peak


def plan_arena(intervals: Sequence[Tuple[int, int, int]]) -> ArenaPlan:
    """`intervals[i] = (bytes, birth, death)`, alive over [birth, death] inclusive.  Returns an offset for each."""
    n = len(intervals)
    sizes = [_align(max(1, b)) for b, _, _ in intervals]
    order = sorted(range(n), key=lambda i: (-sizes[i], -(intervals[i][2] - intervals[i][1]), intervals[i][1]))
    offsets: List[Optional[int]] = [None] * n
    placed: List[int] = []
    reused = 0
    for i in order:
        _, b0, d0 = intervals[i]
        rivals = [j for j in placed if not (intervals[j][2] < b0 or d0 < intervals[j][1])]
        candidates = sorted({0, *(offsets[j] + sizes[j] for j in rivals)})
        for c in candidates:
            if all(c + sizes[i] <= offsets[j] or offsets[j] + sizes[j] <= c for j in rivals):
                offsets[i] = c
                break
        assert offsets[i] is not None  # the end of the highest rival always fits
        if any(offsets[j] < offsets[i] + sizes[i] and offsets[i] < offsets[j] + sizes[j] for j in placed if j not in rivals):
            reused += 1
        placed.append(i)
    peak = max((offsets[i] + sizes[i] for i in range(n)), default=0)
    return ArenaPlan(tuple(offsets), tuple(sizes), peak, n, reused, sum(sizes) - peak)


class Workspace:
    """Hands out step buffers.  `begin(key)` opens a step of capacity bucket `key`; `take`/`give` bracket each
    buffer's life; `end()` closes the step (and, the first time, turns the recording into a plan)."""

    def __init__(self, device, poison: bool = False):
        self.device = device
        self.poison = bool(poison)              # debugging aid: a buffer that is given back is filled with NaN (integers: -1)
        # host-side fault injection (the reference's VELOMIND_FAIL_GRAPH_BUILD_AFTER_ALLOCATIONS, graph_compiler.cpp:562-569):
        # the N-th buffer a step asks for raises instead; the step is abandoned and can be run again
        env = os.environ.get("VELOMIND_B200_FAIL_STEP_AFTER_BUFFERS", "")
        self.fail_after: Optional[int] = int(env) if env.isdigit() else None
        self.arena: Optional[torch.Tensor] = None
        self.generation = 0                     # bumped when the arena moves (captured graphs must be dropped)
        self.plans: Dict[object, ArenaPlan] = {}
        self._key = None
        self._recording = False
        self._log: List[List[int]] = []         # [bytes, birth, death] while recording
        self._live: Dict[int, int] = {}         # data_ptr -> index in the step's take order
        self._clock = 0
        self._next = 0

    def begin(self, key) -> None:
        if self._key is not None:
            raise RuntimeError("Workspace.begin: the previous step was not ended")
        self._key = key
        plan = self.plans.get(key)
        self._recording = plan is None or self.arena is None or self.arena.numel() < plan.peak_bytes
        self._log, self._live, self._clock, self._next = [], {}, 0, 0

    def planned(self, key) -> bool:
        """True if a step of bucket `key` would be served from the arena (its plan exists and fits)."""
        plan = self.plans.get(key)
        return plan is not None and self.arena is not None and self.arena.numel() >= plan.peak_bytes

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        idx = self._next
        if self.fail_after is not None and idx >= self.fail_after:
            raise RuntimeError(f"injected failure: buffer {idx} of the step was refused (fail_after = {self.fail_after})")
        self._next += 1
        self._clock += 1
        if self._recording:
            t = torch.empty(tuple(shape), dtype=dtype, device=self.device)
            self._log.append([nbytes, self._clock, self._clock])
        else:
            plan = self.plans[self._key]
            if idx >= plan.buffer_count or _align(max(1, nbytes)) != plan.sizes[idx]:
                raise RuntimeError(f"Workspace: step of bucket {self._key!r} asks for other buffers than the one it was planned from")
            off = plan.offsets[idx]
            t = self.arena[off: off + nbytes].view(dtype).view(tuple(shape))
        self._live[t.data_ptr()] = idx
        return t

    def give(self, t: Optional[torch.Tensor]) -> None:
        if t is None:
            return
        idx = self._live.pop(t.data_ptr(), None)
        if idx is None:
            raise RuntimeError("Workspace.give: this buffer was not taken in this step (or given twice)")
        self._clock += 1
        if self._recording:
            self._log[idx][2] = self._clock
        if self.poison and t.numel():
            # whoever reads the buffer after this point (a part that gave it back too early, a kernel still to run on
            # it) now reads NaN, and the step's result shows it
            t.fill_(float("nan") if t.dtype.is_floating_point else -1)

    def end(self) -> None:
        if self._live:
            # buffers still held when the step ends live to its end
            for idx in self._live.values():
                if self._recording:
                    self._log[idx][2] = self._clock + 1
        if self._recording:
            plan = plan_arena([tuple(x) for x in self._log])
            self.plans[self._key] = plan
            if self.arena is None or self.arena.numel() < plan.peak_bytes:
                self.arena = None
                self.arena = torch.empty(plan.peak_bytes, dtype=torch.uint8, device=self.device)
                self.generation += 1
        self._key = None
        self._live = {}

    def abort(self) -> None:
        self._key = None
        self._live = {}
