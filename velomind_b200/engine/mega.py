"""The persistent decode kernel's view of a model: one launch per decode step instead of five per layer.

It applies when every layer is pre-norm (RMSNorm) grouped-query attention + SwiGLU with bfloat16 weights of sizes
the weight-streaming kernels take, all layers alike in their sizes, every run owning its cache in one group, a
token-table embedding and a linear head.  The parts describe themselves (`fused_decode_info`); nothing here knows
an architecture's name.  Where it does not apply, decode steps run part by part as before.
"""
from __future__ import annotations

import struct

import torch

from ..kernels import ops

MAX_ROWS = 16


def uniform_layers(model, cache):
    """The layers of `model` as the fused decode kernels see them: (per-run descriptions, the first mixer's, the first
    feed-forward's), if every run is pre-norm (RMSNorm) grouped-query attention + SwiGLU in bfloat16, all alike in
    their sizes, each owning its cache in one unwindowed group.  Raises _NotApplicable otherwise."""
    plan = model.plan
    if model.dtype != torch.bfloat16:
        raise _NotApplicable("compute dtype is not bfloat16")
    if any(e.cache_of is not None for e in plan.schedule):
        raise _NotApplicable("a run reads another run's cache")
    if len(cache.groups) != 1 or cache.groups[0].need.kind != "all":
        raise _NotApplicable("more than one cache group, or a windowed one")
    infos = []
    for entry in plan.schedule:
        block = model.layers[entry.layer].block
        info = getattr(block, "fused_decode_info", lambda: None)()
        if info is None or info["mixer"]["kind"] != "grouped_query_attention" or info["feed_forward"]["kind"] != "swiglu":
            raise _NotApplicable("a layer is not pre-norm attention + SwiGLU in bfloat16")
        infos.append(info)
    m0, f0 = infos[0]["mixer"], infos[0]["feed_forward"]
    keys_m = ("hidden", "heads", "kv_heads", "head_dim", "scale", "window", "rotary_dim")
    for info in infos:
        if any(info["mixer"][k] != m0[k] for k in keys_m) or info["feed_forward"]["intermediate"] != f0["intermediate"]:
            raise _NotApplicable("layers differ in their sizes")
        if info["mixer"]["inv_freq"] is not m0["inv_freq"] and not (
                info["mixer"]["inv_freq"] is not None and m0["inv_freq"] is not None
                and torch.equal(info["mixer"]["inv_freq"], m0["inv_freq"])):
            raise _NotApplicable("layers differ in their rotary frequencies")
    if m0["hidden"] != plan.hidden_size:
        raise _NotApplicable("the mixers' width is not the model's")
    return infos, m0, f0


class MegaPlan:
    def __init__(self, model, cache):
        self.ok = False
        self.why = ""
        self.trace = None          # set to an int64 tensor [phases, CTAs, 2] to record barrier arrival/departure times
        try:
            self._build(model, cache)
        except _NotApplicable as e:
            self.why = str(e)

    def _build(self, model, cache) -> None:
        infos, m0, f0 = uniform_layers(model, cache)
        plan = model.plan
        self.hid, self.H, self.Hkv, self.D = m0["hidden"], m0["heads"], m0["kv_heads"], m0["head_dim"]
        self.I, self.V = f0["intermediate"], plan.vocab_size
        self.scale, self.window, self.rot_dim, self.inv_freq = m0["scale"], m0["window"], m0["rotary_dim"], m0["inv_freq"]
        if (self.hid % 32 or self.I % 32 or (self.H * self.D) % 32 or self.D % 16 or self.D > 64 or self.V % 8
                or self.rot_dim not in (0, self.D) or self.hid != plan.hidden_size):
            raise _NotApplicable("sizes outside what the persistent kernel takes")
        emb, head, fnorm = model.embedding, model.head, model.final_norm
        table = getattr(emb, "table", None)
        head_w = getattr(getattr(head, "proj", None), "weight", None)
        rms = getattr(fnorm, "as_rms", None)
        if table is None or head_w is None or rms is None or head_w.dtype != torch.bfloat16 or table.dtype not in (torch.bfloat16, torch.float32):
            raise _NotApplicable("embedding, final norm or head of another kind")
        self.embed, self.head_w = table, head_w
        self.final_norm, self.final_eps = rms()
        # the per-layer table: 8 pointers and 2 floats per layer, as csrc/decode_mega.cu lays MegaLayer out
        rec = ops.decode_mega_layer_bytes()
        if rec != 8 * 8 + 2 * 4:
            raise _NotApplicable("unexpected layer record size")
        group = cache.groups[0]
        blob = bytearray()
        self._keep = []
        for run, info in enumerate(infos):
            g, li = cache.where(run)
            k, v = group.layer(li)
            n1w, n1e = info["mixer_norm"]
            n2w, n2e = info["feed_forward_norm"]
            ptrs = [info["mixer"]["wqkv"], info["mixer"]["wo"], info["feed_forward"]["wgu"], info["feed_forward"]["wd"], n1w, n2w, k, v]
            self._keep.extend(ptrs)
            blob += struct.pack("<8Q2f", *[t.data_ptr() for t in ptrs], float(n1e), float(n2e))
        self.layers = torch.frombuffer(blob, dtype=torch.uint8).clone().to(model.device)
        self.n_layers = len(infos)
        self.n_pages = group.n_pages
        self.barrier = torch.zeros(1, dtype=torch.int32, device=model.device)
        self.ok = True

    def splits(self, B: int, table_width: int) -> int:
        G = self.H // self.Hkv
        groups = B * self.Hkv * (-(-G // 16))
        return max(1, min(ops.B200_SMS // groups if groups <= ops.B200_SMS else 1, ops.MAX_DECODE_SPLITS, max(1, table_width // 2)))

    def run(self, ctx) -> None:
        """The step of `ctx` (one token per sequence, at most 16 sequences): logits into ctx.logits."""
        B = ctx.B
        table = ctx.tables[0]
        n_splits = self.splits(B, table.shape[1])
        bf = torch.bfloat16
        h = ctx.take((ctx.B_cap, self.hid), torch.float32)
        q = ctx.take((ctx.B_cap, self.H * self.D), bf)
        att = ctx.take((ctx.B_cap, self.H * self.D), bf)
        act = ctx.take((ctx.B_cap, self.I), bf)
        xf = ctx.take((ctx.B_cap, self.hid), bf)
        partial = ctx.take((ctx.B_cap * self.H * ops.MAX_DECODE_SPLITS * (self.D + 2),), torch.float32)
        self.barrier.zero_()
        ops.decode_mega(self.layers, self.n_layers, B, self.hid, self.H, self.Hkv, self.D, self.I, self.V, self.scale, self.window,
                        self.inv_freq, self.rot_dim, ctx.tokens, ctx.positions, ctx.seq_of_token, table, self.n_pages, self.embed,
                        h, q, att, act, xf, ctx.logits, self.final_norm, self.final_eps, self.head_w, partial,
                        ops.decode_counters(ctx.logits.device), n_splits, self.barrier, ctx.err, self.trace)
        for t in (partial, xf, act, att, q, h):
            ctx.ws.give(t)


class _NotApplicable(Exception):
    pass
