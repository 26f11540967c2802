"""Data that describes a model: which parts each layer is made of, and in which order layers run.

An architecture turns its typed configuration into a `ModelPlan`; the engine
builds parts from the plan through the part registries (`parts/registry.py`).
Nothing in here knows an architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry kind and the keyword arguments of its constructor (sizes, eps, theta ...)."""
    kind: str
    args: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class BlockSpec:
    """One layer: an arrangement (how norms, mixer, feed-forward and residual are wired) and its parts.

    `prefix` is the weight-name prefix of this layer in the checkpoint; the
    part prefixes below are relative to it.
    """
    arrangement: str                 # registry kind of the block wiring, e.g. "prenorm"
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    names: Dict[str, str] = field(default_factory=dict)   # part -> sub-prefix, e.g. {"mixer": "self_attn."}


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelPlan.blocks` (a layer may appear several times);
    `cache_of` names the schedule position whose cache this run reads instead of writing its own
    (None: the run owns a cache of its own)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    embedding_prefix: str
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str
    head: PartSpec
    head_prefix: str
    max_positions: int
    stop_tokens: Tuple[int, ...] = ()
    bos_token: Optional[int] = None

    def validate(self) -> None:
        n = len(self.blocks)
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < n:
                raise ValueError(f"schedule[{i}] names layer {e.layer}, the plan has {n}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule[{i}] reads the cache of run {e.cache_of}, which does not come before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}] reads the cache of run {e.cache_of}, which owns none")
