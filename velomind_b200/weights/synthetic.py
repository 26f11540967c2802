"""Random-weights mode: write a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference's `--synthetic` switch fills device buffers with uniform noise
and never writes a file (examples/common/llama/llama_engine.cpp:168-230); here
the random model is an ordinary folder, so everything that reads a model
(engine, replay, tests) takes it through the same loader.

Each tensor draws from its own generator, seeded by (seed, tensor name), so
a tensor's values do not depend on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Optional

import torch

from ..config.base import ConfigError
from ..config.registry import resolve
from .safetensors_io import save_file


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(specs: Dict[str, Any], seed: int, std: float = 0.02, norm_jitter: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """`specs` is the name -> WeightSpec table of a built model.  Matrices and tables get N(0, std);
    vectors flagged `init == "ones"` (norm scales) get 1 + U(-norm_jitter, norm_jitter)."""
    out: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        if spec.alias_of is not None:
            continue  # stored once under the name it aliases
        g = _generator(seed, name)
        if spec.init == "ones":
            t = 1.0 + (torch.rand(spec.shape, generator=g, dtype=torch.float32) * 2.0 - 1.0) * norm_jitter
        elif spec.init == "normal":
            t = torch.randn(spec.shape, generator=g, dtype=torch.float32) * std
        else:
            raise ConfigError(f"tensor {name!r}: unknown init rule {spec.init!r}")
        out[name] = t.to(dtype)
    return out


def write_random_model(folder: str, config: Dict[str, Any], seed: int = 0, std: float = 0.02,
                       norm_jitter: float = 0.1, dtype: str = "bfloat16") -> str:
    """Create `folder` with config.json and model.safetensors for the architecture that `config`
    (a config.json object) names.  Returns the folder."""
    from ..engine.model import weight_table  # late: engine imports weights
    arch = resolve(config, "config")
    typed = arch.config_from_dict(config, "config")
    plan = arch.plan(typed)
    specs = weight_table(plan)
    tdtype = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    tensors = random_tensors(specs, seed, std, norm_jitter, tdtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, indent=2)
        f.write("\n")
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt", "generator": "velomind_b200 random weights", "seed": str(seed)})
    return folder
