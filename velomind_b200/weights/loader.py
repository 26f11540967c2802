"""Weights from safetensors, bound by tensor name and checked against what the model expects.

The model publishes a table `name -> WeightSpec`; `load_weights` reads
`model.safetensors`, and reports everything that does not fit in ONE error:
missing tensors, unexpected tensors, wrong shapes, wrong kinds of dtype.
(The reference checks presence and dtype only, examples/smollm2/model_loader.cpp:115-119,31-34.)

Dtypes stay as stored: a BF16 tensor stays bfloat16, a tensor stored in 32-bit
stays float32, integer tables become int32.  Casting for a compute path is the
business of the part that owns the tensor.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, load_file


class WeightError(ValueError):
    """The tensors of a model folder do not match what the model expects."""


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    kind: str = "float"            # "float": F32/F16/BF16 accepted; "int": an integer table
    init: str = "normal"           # rule of the random-weights mode: "normal" or "ones"
    alias_of: Optional[str] = None  # if the file lacks this tensor, the named tensor stands in (tied head)


def check_and_bind(found: Dict[str, torch.Tensor], specs: Dict[str, WeightSpec], where: str) -> Dict[str, torch.Tensor]:
    missing, wrong_shape, wrong_kind = [], [], []
    bound: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        t = found.get(name)
        if t is None:
            if spec.alias_of is not None and spec.alias_of in found:
                continue  # resolved below, after the target has been checked
            missing.append(name)
            continue
        if tuple(t.shape) != tuple(spec.shape):
            wrong_shape.append(f"{name}: expected {list(spec.shape)}, found {list(t.shape)}")
            continue
        is_float = t.dtype in (torch.float32, torch.float16, torch.bfloat16)
        if (spec.kind == "float") != is_float:
            wrong_kind.append(f"{name}: expected {'a floating-point' if spec.kind == 'float' else 'an integer'} tensor, found {t.dtype}")
            continue
        bound[name] = t
    unexpected = sorted(n for n in found if n not in specs)
    if missing or unexpected or wrong_shape or wrong_kind:
        lines = [f"{where}: the tensors do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if wrong_kind:
            lines.append(f"  wrong dtype ({len(wrong_kind)}): " + "; ".join(wrong_kind))
        raise WeightError("\n".join(lines))
    for name, spec in specs.items():
        if name not in bound:
            bound[name] = bound[spec.alias_of]   # same storage: a tied tensor is really tied
    return bound


def load_weights(folder: str, specs: Dict[str, WeightSpec]) -> Dict[str, torch.Tensor]:
    """Host tensors for every name of `specs`, read from `folder/model.safetensors`."""
    path = os.path.join(folder, "model.safetensors")
    if not os.path.isfile(path):
        hint = ""
        if os.path.isfile(os.path.join(folder, "model.safetensors.index.json")):
            hint = " (a sharded checkpoint with model.safetensors.index.json is not supported; merge the shards)"
        raise WeightError(f"{path}: no such file{hint}")
    try:
        found = load_file(path)
    except SafetensorsError as e:
        raise WeightError(str(e)) from None
    return check_and_bind(found, specs, path)
