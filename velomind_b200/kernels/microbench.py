"""Times one kernel alone at a model's sizes: `python -m velomind_b200.kernels.microbench <kernel> [options]`.

The kernel is launched `--repeat` times in one CUDA graph (as the decode step launches it) and the mean
time per launch is printed with the bytes it has to read and the bandwidth that corresponds to.  Weights
rotate through enough copies to exceed the L2 cache.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from . import ops

KERNELS = ["qkv_rope", "out_residual", "gate_up_swiglu", "down_residual", "head", "attn_decode", "attn_prefill", "attn_prefill_tc", "attn_prefill_ws",
           "add_rmsnorm", "sample", "tc_linear", "tc_residual", "tc_swiglu", "cublas_linear", "prefill_step"]


def _prefill_step(a) -> int:
    """One whole prompt of --tokens tokens through a random model of the given sizes (--layers layers): the step's time
    when replayed from its CUDA graph, and eagerly (the launches one by one, for a launch list under a profiler).  Host clock
    around a call that waits for the device."""
    import tempfile
    import time

    import numpy as np

    from .. import Engine, Entry, load_model, write_random_model
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": a.layers,
           "hidden_size": a.hidden, "num_attention_heads": a.heads, "num_key_value_heads": a.kv_heads,
           "intermediate_size": a.intermediate, "vocab_size": a.vocab, "rope_theta": 100000.0, "rms_norm_eps": 1e-5,
           "tie_word_embeddings": True, "max_position_embeddings": max(8192, a.tokens)}
    T = a.tokens
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, cfg, seed=0)
        model = load_model(d, torch.bfloat16, "cuda:0")
        toks = np.random.default_rng(0).integers(0, a.vocab, size=T).tolist()
        out = {"kernel": "prefill_step", "tokens": T, "layers": a.layers}
        for name, graphs in (("graph", True), ("eager", False)):
            eng = Engine(model, T + 64, use_graphs=graphs)
            times = []
            for _ in range(4 if graphs else 2):
                slot = eng.open()
                eng.synchronize()
                t0 = time.perf_counter()
                eng.step([Entry(slot, toks, [T - 1])])          # waits for the device
                times.append((time.perf_counter() - t0) * 1e3)
                eng.close(slot)
            out[name + "_ms"] = round(min(times), 4)
        print(json.dumps(out))
    return 0


def _time(fn, repeat: int, graph: bool = True) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(repeat):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 5 / repeat * 1e3
    e0.record()
    for _ in range(repeat):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / repeat * 1e3


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kernel", choices=KERNELS)
    ap.add_argument("--batch", type=int, default=8, help="rows (sequences of a decode step)")
    ap.add_argument("--ctx", type=int, default=512, help="cached tokens per sequence (attention kernels)")
    ap.add_argument("--tokens", type=int, default=2048, help="new tokens (attn_prefill)")
    ap.add_argument("--hidden", type=int, default=576)
    ap.add_argument("--heads", type=int, default=9)
    ap.add_argument("--kv-heads", type=int, default=3)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--intermediate", type=int, default=1536)
    ap.add_argument("--vocab", type=int, default=49152)
    ap.add_argument("--n", type=int, default=0, help="tc_*/cublas_linear: output columns (default 2 * intermediate)")
    ap.add_argument("--k", type=int, default=0, help="tc_*/cublas_linear: inner size (default hidden)")
    ap.add_argument("--splits", type=int, default=0, help="attn_decode: key splits (0: the engine's choice)")
    ap.add_argument("--groups", type=int, default=4, help="attn_prefill: warp groups sharing a tile's key blocks")
    ap.add_argument("--cluster", type=int, default=0, help="attn_prefill_ws: CTAs per cluster (0: the launcher's choice)")
    ap.add_argument("--layers", type=int, default=6, help="prefill_step: layers of the random model")
    ap.add_argument("--temp", type=float, default=0.0, help="sample: temperature (0: greedy)")
    ap.add_argument("--top-p", type=float, default=0.9, help="sample: nucleus mass, with --temp")
    ap.add_argument("--variant", type=int, default=0, help="weight-streaming products: 0 the launcher's choice, 1 the register-fed kernel, 2 the one with a ring in shared memory (3 / 4: its form with two pipelines in one CTA / two CTAs per SM)")
    ap.add_argument("--repeat", type=int, default=50)
    ap.add_argument("--no-graph", action="store_true")
    a = ap.parse_args(argv)
    dev = ops.require_cuda("cuda:0")
    ops.skinny_variant(a.variant)
    if a.kernel == "prefill_step":
        return _prefill_step(a)
    M, hid, H, Hkv, D, I, V = a.batch, a.hidden, a.heads, a.kv_heads, a.head_dim, a.intermediate, a.vocab
    bf = torch.bfloat16
    copies = 40
    rot = [0]

    def nxt(ws):
        rot[0] += 1
        return ws[rot[0] % len(ws)]

    h = torch.randn(M, hid, device=dev)
    nw = torch.ones(hid, device=dev)
    x = torch.randn(M, hid, device=dev).to(bf)
    pos = torch.full((M,), a.ctx, dtype=torch.int32, device=dev)
    seq = torch.arange(M, dtype=torch.int32, device=dev)
    width = 1
    while width < a.ctx // 64 + 1:
        width *= 2
    table = torch.arange(M * width, dtype=torch.int32, device=dev).view(M, width)
    n_pages = M * width
    inv = torch.ones(D // 2, device=dev)
    bytes_read = 0
    if a.kernel in ("qkv_rope", "attn_decode", "attn_prefill", "attn_prefill_tc", "attn_prefill_ws"):
        kp = torch.randn(n_pages, Hkv, 64, D, device=dev).to(bf)
        vp = torch.randn_like(kp)
    if a.kernel == "qkv_rope":
        ws = [torch.randn((H + 2 * Hkv) * D, hid, device=dev).to(bf) for _ in range(copies)]
        q = torch.empty(M, H * D, device=dev, dtype=bf)
        fn = lambda: ops.skinny_qkv_rope(h, (nw, 1e-5), nxt(ws), q, pos, seq, table, inv, D, kp, vp, H, Hkv, D)
        bytes_read = ws[0].numel() * 2
    elif a.kernel == "out_residual":
        ws = [torch.randn(hid, H * D, device=dev).to(bf) for _ in range(copies)]
        att = torch.randn(M, H * D, device=dev).to(bf)
        fn = lambda: ops.skinny_linear(att, None, nxt(ws), None, residual=h)
        bytes_read = ws[0].numel() * 2
    elif a.kernel == "gate_up_swiglu":
        ws = [torch.randn(2 * I, hid, device=dev).to(bf) for _ in range(copies)]
        act = torch.empty(M, I, device=dev, dtype=bf)
        fn = lambda: ops.skinny_swiglu(h, (nw, 1e-5), nxt(ws), act)
        bytes_read = ws[0].numel() * 2
    elif a.kernel == "down_residual":
        ws = [torch.randn(hid, I, device=dev).to(bf) for _ in range(copies)]
        act = torch.randn(M, I, device=dev).to(bf)
        fn = lambda: ops.skinny_linear(act, None, nxt(ws), None, residual=h)
        bytes_read = ws[0].numel() * 2
    elif a.kernel == "head":
        ws = [torch.randn(V, hid, device=dev).to(bf) for _ in range(4)]
        logits = torch.empty(M, V, device=dev)
        fn = lambda: ops.skinny_linear(x, None, nxt(ws), logits)
        bytes_read = ws[0].numel() * 2
    elif a.kernel == "attn_decode":
        q = torch.randn(M, H * D, device=dev).to(bf)
        splits = a.splits or ops.decode_splits(M, Hkv, H // Hkv, width)
        partial = torch.empty(M * H * ops.MAX_DECODE_SPLITS * (D + 2), device=dev)
        out = torch.empty(M, H * D, device=dev, dtype=bf)
        fn = lambda: ops.attention_decode_bf16(q, H * D, kp, vp, table, pos, out, partial, ops.decode_counters(dev), H, Hkv, D,
                                               splits, 1.0 / math.sqrt(D))
        bytes_read = M * (a.ctx + 1) * 2 * Hkv * D * 2
    elif a.kernel in ("attn_prefill", "attn_prefill_tc", "attn_prefill_ws"):
        T = a.tokens
        width = 1
        while width < T // 64 + 1:
            width *= 2
        table = torch.arange(width, dtype=torch.int32, device=dev).view(1, width)
        kp = torch.randn(width, Hkv, 64, D, device=dev).to(bf)
        vp = torch.randn_like(kp)
        qkv = torch.randn(T, (H + 2 * Hkv) * D, device=dev).to(bf)
        positions = torch.arange(T, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        out = torch.empty(T, H * D, device=dev, dtype=bf)
        if a.kernel == "attn_prefill_tc":
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda: ops.attention_prefill_tc_bf16(qkv, (H + 2 * Hkv) * D, kp, vp, table, positions, cu, -(-T // 128), out, H, Hkv,
                                                       D, 1.0 / math.sqrt(D), 0, err, a.groups)
        elif a.kernel == "attn_prefill_ws":
            err = torch.zeros(1, dtype=torch.int32, device=dev)
            fn = lambda: ops.attention_prefill_ws_bf16(qkv, (H + 2 * Hkv) * D, kp, vp, table, positions, cu, [0, T], out, H, Hkv,
                                                       D, 1.0 / math.sqrt(D), 0, err, a.cluster)
        else:
            fn = lambda: ops.attention_prefill_bf16(qkv, (H + 2 * Hkv) * D, kp, vp, table, positions, cu, -(-T // 64), out, H, Hkv, D,
                                                    1.0 / math.sqrt(D), groups=a.groups)
        bytes_read = 0
    elif a.kernel in ("tc_linear", "tc_residual", "tc_swiglu", "cublas_linear"):
        T, N, K = a.tokens, a.n or 2 * I, a.k or hid
        xs = torch.randn(T, K, device=dev).to(bf)
        ws = [torch.randn(N, K, device=dev).to(bf) for _ in range(8)]
        outb = torch.empty(T, N, device=dev, dtype=bf)
        hres = torch.zeros(T, N, device=dev)
        act = torch.empty(T, N // 2, device=dev, dtype=bf)
        if a.kernel == "tc_linear":
            fn = lambda: ops.tc_linear(xs, nxt(ws), outb)
        elif a.kernel == "tc_residual":
            fn = lambda: ops.tc_linear(xs, nxt(ws), None, residual=hres)
        elif a.kernel == "tc_swiglu":
            fn = lambda: ops.tc_swiglu(xs, nxt(ws), act)
        else:
            fn = lambda: torch.mm(xs, nxt(ws).t(), out=outb)
        bytes_read = 0
        flops_mm = 2.0 * T * N * K
    elif a.kernel == "add_rmsnorm":
        out = torch.empty(M, hid, device=dev, dtype=bf)
        fn = lambda: ops.add_rmsnorm(h, None, nw, 1e-5, out)
        bytes_read = M * hid * 4
    else:
        logits = torch.randn(M, V, device=dev) * 3.0
        out = torch.empty(M, dtype=torch.int32, device=dev)
        if a.temp > 0:
            temps = torch.full((M,), a.temp, device=dev)
            tps = torch.full((M,), a.top_p, device=dev)
            seeds = torch.full((M,), 42, dtype=torch.int64, device=dev)
            ids = torch.arange(M, dtype=torch.int64, device=dev)
            fn = lambda: ops.sample(logits, temps, tps, seeds, ids, ids, out)
        else:
            fn = lambda: ops.sample(logits, None, None, None, None, None, out)
        bytes_read = M * V * 4
    us = _time(fn, a.repeat, graph=not a.no_graph)
    res = {"kernel": a.kernel, "rows": M, "us_per_launch": round(us, 3), "bytes_read": bytes_read,
           "GB_per_s": round(bytes_read / us / 1e3, 1) if bytes_read else None}
    if a.kernel in ("tc_linear", "tc_residual", "tc_swiglu", "cublas_linear"):
        res["rows"] = a.tokens
        res["TFLOP_per_s"] = round(flops_mm / us / 1e6, 1)
    if a.kernel == "attn_prefill":
        flops = 4.0 * D * H * a.tokens * (a.tokens + 1) / 2
        res["TFLOP_per_s"] = round(flops / us / 1e6, 1)
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
