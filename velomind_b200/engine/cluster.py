"""The cluster decode kernel's view of a model: embedding and all layers of a decode step in one launch.

The sequences of a decode batch do not depend on one another, so the batch is dealt out to thread-block clusters
that each take a few sequences through every layer without any synchronisation across the grid
(csrc/decode_cluster.cu).  The kernel's input is a stream: for every layer and every CTA rank of a cluster, the
weights that rank multiplies with, in the order it needs them, already arranged as tensor-core operand fragments.
This module packs that stream once per model (a second copy of the layers' weights in device memory) and decides,
per step shape, how many sequences a cluster takes and into how many parts the attention over a sequence is cut.

It applies to the same models as the persistent kernel of engine/mega.py (pre-norm RMSNorm + grouped-query
attention + SwiGLU layers, all alike, bfloat16); the parts describe themselves through `fused_decode_info`, and
nothing here knows an architecture's name.  The final norm and the head run as the model's own parts.
"""
from __future__ import annotations

import struct
from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .mega import _NotApplicable, uniform_layers

CLUSTER_SIZE = 16          # CTAs per cluster (the largest the hardware takes)
MAX_CLUSTERS = 4           # clusters of 16 CTAs seen running at once on a B200: a batch is dealt out to at most this many
MAX_ROWS_PER_CLUSTER = 16
KS_TARGET = 3              # k32 blocks of a warp's 16-row weight tile per ring stage, at most: 8 warps x 3 x 1 KB = 24 KB a stage


def choose_split(n_units: int, ksteps: int, ks_target: int = KS_TARGET) -> Tuple[int, int, int, int, int]:
    """How a rank's `n_units` units of a product with `ksteps` k32 blocks are dealt out to the kernel's eight consumer
    warps: (ksplit warps per unit, ks steps per warp and ring stage, units per round, rounds, stages per round).
    The same rule, integer for integer, as choose_split in csrc/decode_cluster.cu."""
    best, best_cost = (1, 1, 8, 0, 0), -1
    ksplit = 1
    while ksplit <= 8:
        if ksteps % ksplit == 0:
            per, upr = ksteps // ksplit, 8 // ksplit
            ks = max(d for d in range(1, min(ks_target, per) + 1) if per % d == 0)
            rounds = -(-n_units // upr)
            cost = rounds * (per + 2 * (per // ks) + 16)
            if best_cost < 0 or cost < best_cost:
                best, best_cost = (ksplit, ks, upr, rounds, per // ks), cost
        ksplit *= 2
    return best


def _fragments(w: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """Weight rows `rows` [units, 16] of w [N, K] (bfloat16) as mma.sync m16n8k16 A fragments, two per k32 block:
    [units, K/32, 512], the 512 values of a (unit, block) being 2 steps x 32 lanes x (a0, a1, a2, a3) x 2, lane = 4 g + q.
    Inside a block the k order is permuted so that lane q's B operands of BOTH steps are the eight consecutive values
    x[32 s + 8 q ..] of an activation row (one 16-byte load): step j of block s multiplies
    a0 = w[row g, 32 s + 8 q + 4 j + (0, 1)], a2 = w[row g, 32 s + 8 q + 4 j + (2, 3)], a1 and a3 the same of row g + 8."""
    n, K = rows.shape[0], w.shape[1]
    x = w[rows.reshape(-1)].reshape(n, 2, 8, K // 32, 4, 2, 2, 2)        # [unit, half, g, block, q, step, khalf, e]
    return x.permute(0, 3, 5, 2, 4, 6, 1, 7).reshape(n, K // 32, 512)    # [unit, block, step, g, q, khalf, half, e]


def _stages(frags: torch.Tensor) -> torch.Tensor:
    """The fragments [units, blocks, 512] of one rank's units in the order its warps consume them: rounds of a few
    units, `ksplit` warps sharing a unit's k32 blocks, each round cut along K into stages of `ks` blocks per warp; a
    stage is [units of the round][ksplit][ks][512]."""
    n, steps, _ = frags.shape
    ksplit, ks, upr, rounds, chunks = choose_split(n, steps)
    out = []
    for rd in range(rounds):
        part = frags[rd * upr:(rd + 1) * upr]
        out.append(part.reshape(part.shape[0], ksplit, chunks, ks, 512).permute(2, 0, 1, 3, 4).reshape(-1))
    return torch.cat(out) if out else frags.new_zeros(0)


def _bytes(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8).reshape(-1)


class ClusterPlan:
    def __init__(self, model, cache, cluster_size: int = CLUSTER_SIZE):
        self.ok = False
        self.why = ""
        self.cs = int(cluster_size)
        self._shapes: Dict[Tuple[int, int], Optional[Tuple[int, int]]] = {}
        self.trace = None          # set to an int64 tensor [5 * layers, CTAs, 2] to record the phase barriers' times
        self.last_shape: Optional[Tuple[int, int]] = None     # (sequences per cluster, attention parts) of the last step
        try:
            self._build(model, cache)
        except _NotApplicable as e:
            self.why = str(e)

    # ---- once per model
    def _build(self, model, cache) -> None:
        infos, m0, f0 = uniform_layers(model, cache)
        plan = model.plan
        self.model = model
        self.hid, self.H, self.Hkv, self.D = m0["hidden"], m0["heads"], m0["kv_heads"], m0["head_dim"]
        self.I, self.V = f0["intermediate"], plan.vocab_size
        self.scale, self.window, self.rot_dim, self.inv_freq = m0["scale"], m0["window"], m0["rotary_dim"], m0["inv_freq"]
        hid, H, Hkv, D, I = self.hid, self.H, self.Hkv, self.D, self.I
        if (D not in (16, 32, 64, 128) or hid % 32 or (H * D) % 32 or I % 32 or H % Hkv or H // Hkv > 16
                or self.rot_dim not in (0, D)):
            raise _NotApplicable("sizes outside what the cluster kernel takes")
        table = getattr(model.embedding, "table", None)
        if table is None or table.dtype not in (torch.bfloat16, torch.float32) or not hasattr(model, "finish"):
            raise _NotApplicable("embedding of another kind")
        self.embed = table
        if ops.decode_cluster_layer_bytes() != 3 * 8 + 2 * 4:
            raise _NotApplicable("unexpected layer record size")
        if ops.decode_cluster_fit(1, self.cs, len(infos), hid, H, Hkv, D, I, 1, KS_TARGET, 1) < 3:
            raise _NotApplicable("the rows' activations leave no shared memory for the weight ring")
        dev = model.device
        cs = self.cs
        idx = lambda *a: torch.arange(*a, device=dev)
        # the 16 weight rows of each unit (two runs of 8), per product
        u = idx((H + 2 * Hkv) * D // 16)
        first = (u // (D // 16)) * D + (u % (D // 16)) * 8                  # head * D + d0: pairs (d, d + D/2) share a thread
        rows_qkv = torch.cat([first[:, None] + idx(8)[None], first[:, None] + D // 2 + idx(8)[None]], 1)
        rows_out = idx(hid // 16)[:, None] * 16 + idx(16)[None]
        g0 = idx(I // 8)[:, None] * 8 + idx(8)[None]
        rows_gu = torch.cat([g0, I + g0], 1)                                # gate rows, then the up rows of the same columns
        split = lambda n, c: (n * c // cs, n * (c + 1) // cs)
        group = cache.groups[0]
        packed, blob = [], bytearray()
        for run, info in enumerate(infos):
            mx, ff = info["mixer"], info["feed_forward"]
            n1w, n1e = info["mixer_norm"]
            n2w, n2e = info["feed_forward_norm"]
            f_qkv = _fragments(mx["wqkv"], rows_qkv)
            f_out = _fragments(mx["wo"], rows_out)
            f_gu = _fragments(ff["wgu"], rows_gu)
            f_down = _fragments(ff["wd"], rows_out)
            ranks = []
            for c in range(cs):
                a, b = split(f_qkv.shape[0], c)
                o0, o1 = split(f_out.shape[0], c)
                g_a, g_b = split(f_gu.shape[0], c)
                ranks.append(torch.cat([
                    _bytes(n1w.float()), _bytes(_stages(f_qkv[a:b])), _bytes(_stages(f_out[o0:o1])),
                    _bytes(n2w.float()), _bytes(_stages(f_gu[g_a:g_b])), _bytes(_stages(f_down[o0:o1]))]))
            stride = -(-max(r.numel() for r in ranks) // 128) * 128
            layer = torch.zeros((cs, stride), dtype=torch.uint8, device=dev)
            for c, r in enumerate(ranks):
                layer[c, : r.numel()] = r
            packed.append(layer)
        self.rank_stride = max(p.shape[1] for p in packed)
        self.stream = torch.zeros((len(packed), cs, self.rank_stride), dtype=torch.uint8, device=dev)
        for i, layer in enumerate(packed):
            self.stream[i, :, : layer.shape[1]] = layer
        del packed
        self._keep = []
        for run, info in enumerate(infos):
            g, li = cache.where(run)
            k, v = group.layer(li)
            self._keep.extend([k, v])
            blob += struct.pack("<3Q2f", self.stream[run].data_ptr(), k.data_ptr(), v.data_ptr(),
                                float(info["mixer_norm"][1]), float(info["feed_forward_norm"][1]))
        self.layers = torch.frombuffer(blob, dtype=torch.uint8).clone().to(dev)
        self.n_layers = len(infos)
        self.n_pages = group.n_pages
        self.ok = True

    # ---- once per step shape
    def shape_for(self, B: int, table_width: int) -> Optional[Tuple[int, int]]:
        """(sequences per cluster, attention parts per (sequence, kv head)) for a batch of B sequences whose block
        tables are `table_width` wide, or None if the kernel does not take this shape."""
        key = (B, table_width)
        if key not in self._shapes:
            self._shapes[key] = self._choose(B, table_width)
        return self._shapes[key]

    def _choose(self, B: int, table_width: int) -> Optional[Tuple[int, int]]:
        rows = -(-B // MAX_CLUSTERS)
        rows = -(-B // -(-B // rows))          # the same number of clusters, as even as possible
        if rows > MAX_ROWS_PER_CLUSTER:
            return None
        parts = max(1, min(self.cs // (rows * self.Hkv), table_width))
        while parts >= 1:
            if ops.decode_cluster_fit(rows, self.cs, self.n_layers, self.hid, self.H, self.Hkv, self.D, self.I, table_width,
                                      KS_TARGET, parts) >= 3:
                return rows, parts
            parts //= 2
        return None

    def takes(self, ctx) -> bool:
        return self.ok and ctx.one_token_each and self.shape_for(ctx.B, ctx.tables[0].shape[1]) is not None

    def run(self, ctx) -> None:
        """The step of `ctx` (one new token per sequence): logits of the wanted rows into ctx.logits."""
        table = ctx.tables[0]
        rows, parts = self.last_shape = self.shape_for(ctx.B, table.shape[1])
        h = ctx.take_tokens(self.hid, torch.float32)
        ops.decode_cluster(self.layers, self.n_layers, ctx.B, rows, self.cs, self.hid, self.H, self.Hkv, self.D, self.I, self.V,
                           self.scale, self.window, self.inv_freq, self.rot_dim, ctx.tokens, ctx.positions, table, self.n_pages,
                           self.embed, h, self.rank_stride, KS_TARGET, parts, ctx.err, self.trace)
        self.model.finish(ctx, h, None)
