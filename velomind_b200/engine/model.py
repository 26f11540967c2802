"""A decoder model built from a plan: embedding, layers run in the plan's order, final norm, head.

Nothing here names an architecture; the plan says which parts and which order.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops

from ..cache.store import CacheNeed
from ..config.base import read_config_json
from ..config.registry import resolve
from ..parts.base import BindContext
from ..parts.registry import build_part
from ..parts.spec import ModelPlan, PartSpec
from ..weights.loader import WeightSpec, load_weights


class Layer:
    """The parts of one layer and its wiring, plus the weight-name prefix of each part."""

    def __init__(self, spec):
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.feed_forward = build_part("feed_forward", spec.feed_forward)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.feed_forward_norm = build_part("norm", spec.feed_forward_norm)
        self.block = build_part("arrangement", PartSpec(spec.arrangement, {
            "mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
            "feed_forward_norm": self.feed_forward_norm}))

    def named_parts(self):
        for role in ("mixer", "feed_forward", "mixer_norm", "feed_forward_norm"):
            yield self.spec.prefix + self.spec.names.get(role, role + "."), getattr(self, role)


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.layers: List[Layer] = [Layer(b) for b in plan.blocks]
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.dtype: Optional[torch.dtype] = None
        self.device = None

    # ---- weights
    def named_parts(self):
        yield self.plan.embedding_prefix, self.embedding
        for layer in self.layers:
            yield from layer.named_parts()
        yield self.plan.final_norm_prefix, self.final_norm
        yield self.plan.head_prefix, self.head

    def weight_table(self) -> Dict[str, WeightSpec]:
        table: Dict[str, WeightSpec] = {}
        for prefix, part in self.named_parts():
            for name, spec in part.weight_specs().items():
                table[prefix + name] = spec
        return table

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """Put the host tensors (names of `weight_table`) on `device` for compute dtype `dtype`."""
        ops.require_cuda(device)                 # (one clear refusal before the first tensor moves: there is no CPU fallback)
        bc = BindContext(dtype, torch.device(device))
        for prefix, part in self.named_parts():
            part.bind({name: tensors[prefix + name] for name in part.weight_specs()}, bc)
        self.dtype, self.device = dtype, torch.device(device)

    @property
    def graph_safe(self) -> bool:
        """True if every part says its decode step may be recorded into a CUDA graph."""
        parts = [p for _, p in self.named_parts()] + [l.block for l in self.layers]
        parts += [l.mixer.position for l in self.layers if hasattr(l.mixer, "position")]
        return all(getattr(p, "graph_safe", False) for p in parts)

    # ---- cache needs, one per schedule position
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        out: List[Optional[CacheNeed]] = []
        for entry in self.plan.schedule:
            mixer = self.layers[entry.layer].mixer
            out.append(None if entry.cache_of is not None else mixer.cache_need())
        return out

    def cache_shares(self) -> List[Optional[int]]:
        return [e.cache_of for e in self.plan.schedule]

    # ---- one step
    def forward(self, ctx) -> torch.Tensor:
        """Run the step's tokens through every layer of the schedule; float32 logits [R, vocab] at ctx.logit_rows."""
        hid = self.plan.hidden_size
        h = ctx.take_tokens(hid, torch.float32)
        self.embedding.forward(ctx, ctx.tokens, h)
        pending = None
        for run, entry in enumerate(self.plan.schedule):
            ctx.run = run
            pending = self.layers[entry.layer].block.forward(ctx, h, pending)
        ctx.run = None
        return self.finish(ctx, h, pending)

    def finish(self, ctx, h: torch.Tensor, pending) -> torch.Tensor:
        """Final norm and head on the wanted rows of the residual stream `h` (plus `pending`, a product not yet added
        to it); gives `h` and `pending` back to the workspace."""
        hid = self.plan.hidden_size
        logits = ctx.logits
        # (the buffer is taken whatever R is, so that every step of a capacity bucket asks for the same buffers; it is
        # given back by its whole extent: with R = 0, a prompt cut into several steps, the view of its rows is empty)
        rows = ctx.take((ctx.R_cap, hid), ctx.act_dtype)
        if ctx.R > 0:
            x = rows[: ctx.R]
            self.final_norm.forward(ctx, h, pending, x, ctx.logit_rows)
            self.head.forward(ctx, x, logits)
        ctx.ws.give(rows)
        ctx.ws.give(pending)
        ctx.ws.give(h)
        return logits


def weight_table(plan: ModelPlan) -> Dict[str, WeightSpec]:
    return DecoderModel(plan).weight_table()


def load_model(folder: str, dtype: torch.dtype, device) -> DecoderModel:
    """Read config.json, choose the architecture by its name, build the parts, load and bind the weights."""
    data = read_config_json(folder)
    arch = resolve(data, f"{folder}/config.json")
    config = arch.config_from_dict(data, f"{folder}/config.json")
    model = DecoderModel(arch.plan(config))
    model.config = config
    tensors = load_weights(folder, model.weight_table())
    model.bind(tensors, dtype, device)
    return model
