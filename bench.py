"""Decode and prefill throughput of the library on one B200, at the sizes of SmolLM2-135M with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 (prompts of 512 tokens, cache sized
for context 4096), timed on the device with CUDA events over exactly K decode steps, each of which runs
the step function and the device sampler and hands the tokens to the host.  `e2e` is the same through
`TextEngine.generate` (host token ids in, host token ids out, wall clock of its decode steps).  `prefill`
is one prompt of 2,048 tokens; `points` holds decode at batch 1 and 64; `roofline` compares the decode
step with the bytes it has to read.  The reference publishes no number (`vs_baseline` is null).

`--impl reference` runs the UNMODIFIED reference, built by baseline/build_reference.py into baseline/_ref (its core,
its CUDA backend and its own benchmark tool; pip cannot install it, it is a CMake project without a Python package):
`value` and `prefill` come from its own `benchmark_baseline --device cuda --synthetic` (one execute of its decode
graph at context 512, one execute of its 2,048-token prompt graph: benchmarks/benchmark_runner.cpp:134-158,190-249),
`e2e` from its public engine API (`prefill` + `forward_step`, host tokens in, host logits out, graph build and
allocation of every step included, as its own generation loop pays them).  The reference runs one sequence at a time:
its batch of 8 is eight sequences one after another, so its tokens per second do not grow with the batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# other shapes of the family (config.json keys that differ from the 135M sizes): the benchmark itself is the 135M shape
SHAPES = {
    "135m": {},
    "360m": {"num_hidden_layers": 32, "hidden_size": 960, "num_attention_heads": 15, "num_key_value_heads": 5,
             "intermediate_size": 2560},
    "1.7b": {"num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 32,
             "intermediate_size": 8192, "rope_theta": 130000.0},
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS)
    src = "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                data = json.load(f)
            for k in out:
                if isinstance(data.get(k), (int, float)) and data[k] > 0:
                    out[k] = float(data[k])
                    src = "measured"
        except (OSError, ValueError):
            pass
    out["source"] = src
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: NVML read every two milliseconds from a thread
    (reads only; nothing is set), or nvidia-smi every 100 ms where the NVML binding is missing."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self):
        self.proc = None
        self.lines = []
        self.nvml = None
        self.handle = None
        self.samples = []           # (sm MHz, reason bits)
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(os.environ.get("LOCAL_RANK", "0")))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.stop_flag.clear()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag.is_set():
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)), int(reasons_fn(self.handle))))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            if self.thread:
                self.thread.join(timeout=1.0)
            sm = [s for s, _ in self.samples]
            reasons = sorted(n for n, bit in self.REASON_BITS.items() if any(r & bit for _, r in self.samples))
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(sm),
                    "source": "nvml, every 2 ms"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi, every 100 ms"}


def model_bytes_and_flops(cfg, layers):
    hid, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = hid // H
    per_layer = hid * (H + 2 * Hkv) * D + H * D * hid + 3 * hid * I       # matrix elements of one layer
    norms = (2 * layers + 1) * hid
    weight_bytes = 2 * (per_layer * layers + V * hid) + 4 * norms          # bf16 matrices (tied head read once), f32 norms
    kv_bytes_per_token = 2 * Hkv * D * 2 * layers
    return per_layer, weight_bytes, kv_bytes_per_token, D


def decode_run(text_engine, B, prompt_len, steps, warmup, vocab, clock=None, context_fill=0):
    """K timed decode steps at batch B; returns (ms per step, mean context, own-kernel launches, library calls, clocks).
    Timed on the device: CUDA events on the engine's own stream around exactly K steps, each of which runs the step function,
    the device sampler and the token feedback."""
    import numpy as np
    import torch
    from velomind_b200 import Entry, SamplingParams
    eng = text_engine.engine
    stream = eng.stream
    rng = np.random.default_rng(B)
    slots = [eng.open() for _ in range(B)]
    params = [SamplingParams(temperature=0.0)] * B
    streams = list(range(B))
    first = context_fill or prompt_len
    logits = eng.step([Entry(s, rng.integers(0, vocab, first).tolist(), [first - 1]) for s in slots])
    toks = eng.sample(logits, params, streams, [0] * B)
    state = {"toks": toks, "done": 1}

    def run(k):
        # k decode steps queued on the GPU: forward, device sampler and token feedback per step, no host in between
        rows = eng.decode_many(slots, state["toks"], params, streams, [state["done"]] * B, k)
        state["toks"], state["done"] = rows[-1], state["done"] + k

    done = 0
    while done < warmup:
        k = min(eng.MAX_DECODE_RUN, warmup - done)
        run(k)
        done += k
    run(min(eng.MAX_DECODE_RUN, steps))          # the shape of the timed run, recorded before the clock starts
    eng.synchronize()
    ctx0 = eng.length(slots[0])
    c0 = eng.counters
    if clock:
        clock.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    done = 0
    while done < steps:
        k = min(eng.MAX_DECODE_RUN, steps - done)
        run(k)
        done += k
    ev1.record(stream)
    eng.synchronize()
    clocks = clock.stop() if clock else None
    ms = ev0.elapsed_time(ev1) / steps
    c1 = eng.counters
    launches, calls = c1["own_launches"] - c0["own_launches"], c1["library_calls"] - c0["library_calls"]
    mean_ctx = ctx0 + (steps + 1) / 2.0
    for s in slots:
        eng.close(s)
    eng.raise_if_error()
    return ms, mean_ctx, launches, calls, clocks


def prefill_run(engine, T, vocab, repeats=5):
    """Median device time of one whole prompt of T tokens (with the head on its last row): CUDA events on the engine's stream."""
    import numpy as np
    import torch
    from velomind_b200 import Entry
    rng = np.random.default_rng(7)
    stream = engine.stream
    times = []
    for r in range(repeats + 2):
        toks = rng.integers(0, vocab, T).tolist()
        slot = engine.open()
        engine.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        engine.step([Entry(slot, toks, [T - 1])], synchronize=False)
        ev1.record(stream)
        engine.synchronize()
        engine.close(slot)
        if r >= 2:
            times.append(ev0.elapsed_time(ev1))
    engine.raise_if_error()
    return statistics.median(times)


def unequal_batch_run(text_engine, batch, lo, hi, decode_steps, vocab):
    """BASELINE.json's 360M run: `batch` prompts of lengths uniform in [lo, hi], then `decode_steps` tokens each through the
    public entry point; returns (decoded tokens per second, prompt tokens per second, prompt tokens)."""
    import numpy as np
    rng = np.random.default_rng(16)
    prompts = [rng.integers(0, vocab, int(n)).tolist() for n in rng.integers(lo, hi + 1, batch)]
    text_engine.generate(prompts, temperature=0.0, max_tokens=4, stop_tokens=())          # warm-up: plans and graphs of these shapes
    text_engine.generate(prompts, temperature=0.0, max_tokens=decode_steps + 1, stop_tokens=())
    tm = text_engine.last_timing
    n_prompt = sum(len(p) for p in prompts)
    return batch * tm.decode_steps / tm.decode_seconds, n_prompt / tm.prefill_seconds, n_prompt


def _parse_reference_table(markdown: str):
    """Rows of the reference tool's report: {S: (prefill ms, prefill tok/s, decode ms, decode tok/s)} of the CUDA backend."""
    rows = {}
    for line in markdown.splitlines():
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) < 8 or cells[0] != "CUDA":
            continue
        try:
            S = int(cells[1])
            prefill_ms = float(cells[4].split("/")[0])
            prefill_tps = float(cells[5].split()[0])
            decode_ms = float(cells[6].split("/")[0])
            decode_tps = float(cells[7].split()[0])
        except (ValueError, IndexError):
            continue
        rows[S] = (prefill_ms, prefill_tps, decode_ms, decode_tps)
    return rows


def reference_arm(args):
    """The reference's own numbers for the same metric and sizes, or the one-line reason why there are none."""
    if args.gpus != 1:
        return {"impl": "reference", "unavailable": "the reference runs on one device only"}
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    tool, driver = os.path.join(ref_dir, "benchmark_baseline"), os.path.join(ref_dir, "reference_driver")
    if not (os.path.isfile(tool) and os.path.isfile(driver)):
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import build_reference
            build_reference.build()
        except Exception as ex:      # no checkout of the reference, or no compiler
            return {"impl": "reference", "unavailable": f"the reference could not be built here: {str(ex).splitlines()[0][:200]}"}
    B, prompt_len, T = 8, 512, 2048
    steps, warmup = max(1, args.steps), max(args.warmup, 3)
    clock = ClockSampler()
    with tempfile.TemporaryDirectory(prefix="velomind_ref_") as work:
        report = os.path.join(work, "report.md")
        clock.start()
        # its own tool: median over `steps` executes after `warmup`; S = 512 gives decode at context 512, S = 2048 the prompt
        r = subprocess.run([tool, "--device", "cuda", "--synthetic", "--seq-lens", f"{prompt_len},{T}", "--iters", str(min(steps, 20)),
                            "--warmup", str(warmup), "--quiet", "--markdown", report], cwd=work, capture_output=True, text=True, timeout=1500)
        clocks = clock.stop()
        if r.returncode != 0 or not os.path.isfile(report):
            return {"impl": "reference", "unavailable": f"the reference's benchmark tool failed (exit {r.returncode}): {(r.stderr or r.stdout).strip().splitlines()[-1][:200] if (r.stderr or r.stdout).strip() else ''}"}
        with open(report) as f:
            rows = _parse_reference_table(f.read())
        if prompt_len not in rows or T not in rows:
            return {"impl": "reference", "unavailable": "the reference's report has no CUDA rows (no CUDA device?)"}
        # end to end through its public engine API: B sequences one after another, host tokens in, host logits out
        d = subprocess.run([driver, "cuda", str(B), str(prompt_len), str(min(steps, 20)), "3", str(T)], cwd=work, capture_output=True,
                           text=True, timeout=1500)
        e2e = None
        if d.returncode == 0:
            try:
                rec = json.loads(d.stdout.strip().splitlines()[-1])
                n = rec["sequences"] * rec["decode_steps"]
                e2e = {"value": n * 1000.0 / rec["decode_ms_total"], "unit": "tokens/s", "h2d_bytes_per_step": 4,
                       "d2h_bytes_per_step": rec["logit_bytes_per_step"], "ms_per_token": rec["decode_ms_median"],
                       "prefill_2048_ms": rec["prefill_ms_median"]}
            except (ValueError, KeyError, IndexError):
                e2e = None
    _, _, decode_ms, decode_tps = rows[prompt_len]
    prefill_ms, prefill_tps, _, _ = rows[T]
    pk = peaks()
    cfg = {"hidden_size": 576, "intermediate_size": 1536, "vocab_size": 49152, "num_attention_heads": 9, "num_key_value_heads": 3}
    per_layer, _, _, D = model_bytes_and_flops(cfg, 30)
    flops = 2.0 * T * per_layer * 30 + 4.0 * D * 9 * (T * (T + 1) / 2.0) * 30 + 2.0 * 49152 * 576
    line = {
        "impl": "reference",
        "metric": "decode tok/s at batch 8 (SmolLM2-135M shape, prompts of 512 tokens)",
        "value": decode_tps, "unit": "tokens/s", "n_gpus": 1, "steps": min(steps, 20), "warmup": warmup,
        "ms_per_step": decode_ms * B, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic",
        "config": {"model": "SmolLM2-135M shape, the reference's own --synthetic weights", "global_batch": B, "seq_len": prompt_len,
                   "parallelism": "single GPU", "layers": 30, "layers_of_config": 30, "hidden": 576, "heads": 9, "kv_heads": 3,
                   "head_dim": 64, "intermediate": 1536, "vocab": 49152,
                   "batching": "none in the reference: 8 sequences one after another, tokens/s equal its batch-1 figure",
                   "timing": "the reference's own tool: host clock around one execute of its decode graph, median",
                   "built_from": "unmodified sources, CUDA backend for sm_100, cuBLAS float32"},
        "prefill": {"value": prefill_tps, "tokens": T, "ms": prefill_ms, "frac": flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)},
        "points": {"decode_b1": decode_tps, "decode_b64": decode_tps},
        "clocks": clocks,
        "gpu_launches": 0,
    }
    if e2e is not None:
        line["e2e"] = e2e
    return line


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all); reported in config")
    ap.add_argument("--quick", action="store_true", help="skip the batch 1 / 64 points and the end-to-end run")
    ap.add_argument("--shape", default="135m", choices=sorted(SHAPES),
                    help="sizes of the random model: the benchmark's SmolLM2-135M (default), or the 360M / 1.7B shapes of the family")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps(reference_arm(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU library: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    warmup = max(args.warmup, 3)

    import numpy as np
    import velomind_b200 as vm

    cfg = dict(vm.SMOLLM2_135M)
    cfg.update(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    vocab = cfg["vocab_size"]
    B, prompt_len, context = 8, 512, 4096
    pk = peaks()

    with tempfile.TemporaryDirectory(prefix="velomind_bench_") as folder:
        vm.write_random_model(folder, cfg, seed=0, std=0.02)
        te = vm.TextEngine(vm.EngineConfig(model_path=folder, dtype="bfloat16", max_tokens=64 * context + 8192, max_batch=64)).load()

    per_layer, weight_bytes, kv_per_token, D = model_bytes_and_flops(cfg, layers)

    clock = ClockSampler()
    ms, mean_ctx, launches, calls, clocks = decode_run(te, B, prompt_len, args.steps, warmup, vocab, clock)
    value = B * 1000.0 / ms
    step_bytes = weight_bytes + kv_per_token * mean_ctx * B
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # prefill of 2,048 tokens: linears + causal attention + the head on one row.  The headline figure is a FIRST-SEEN shape: the
    # step's kernels launched one by one from the host, which is what a prompt of a new length gets; the same step replayed from
    # its CUDA graph (what a repeated shape gets) goes to `points`.
    T = 2048
    fresh = vm.Engine(te.model, T + 64, use_graphs=False)
    pms = prefill_run(fresh, T, vocab)
    del fresh
    H = cfg["num_attention_heads"]
    flops = 2.0 * T * per_layer * layers + 4.0 * D * H * (T * (T + 1) / 2.0) * layers + 2.0 * vocab * cfg["hidden_size"]
    prefill = {"value": T * 1000.0 / pms, "tokens": T, "ms": pms, "frac": flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    points, e2e = {}, None
    if not args.quick:
        replayed_ms = prefill_run(te.engine, T, vocab)
        points["prefill_2048_replayed"] = T * 1000.0 / replayed_ms
        for b in (1, 64):
            m, _, _, _, _ = decode_run(te, b, prompt_len, args.steps, warmup, vocab)
            points[f"decode_b{b}"] = b * 1000.0 / m
        # end to end through the public entry point: host token ids in, host token ids out
        rng = np.random.default_rng(1)
        prompts = [rng.integers(0, vocab, prompt_len).tolist() for _ in range(B)]
        # the host reads every step's tokens and sends the next step's descriptors (steps_per_sync=1), as the contract asks
        te.generate(prompts, temperature=0.0, max_tokens=warmup + 1, stop_tokens=(), steps_per_sync=1)
        # bytes are counted where they are copied (descriptors and sampler parameters up, sampled tokens down); what the
        # prompt step alone moves is taken off, as the timed region is the decode steps
        c0 = te.engine.counters
        te.generate(prompts, temperature=0.0, max_tokens=1, stop_tokens=(), steps_per_sync=1)
        c1 = te.engine.counters
        h2d_prompt, d2h_prompt = c1["h2d_bytes"] - c0["h2d_bytes"], c1["d2h_bytes"] - c0["d2h_bytes"]
        te.generate(prompts, temperature=0.0, max_tokens=args.steps + 1, stop_tokens=(), steps_per_sync=1)
        c2 = te.engine.counters
        tm = te.last_timing
        e2e = {"value": B * tm.decode_steps / tm.decode_seconds, "unit": "tokens/s",
               "h2d_bytes_per_step": round((c2["h2d_bytes"] - c1["h2d_bytes"] - h2d_prompt) / max(tm.decode_steps, 1)),
               "d2h_bytes_per_step": round((c2["d2h_bytes"] - c1["d2h_bytes"] - d2h_prompt) / max(tm.decode_steps, 1))}
        # the same call with 8 decode steps queued per host round trip
        te.generate(prompts, temperature=0.0, max_tokens=args.steps + 1, stop_tokens=(), steps_per_sync=8)
        points["e2e_queued_8"] = B * te.last_timing.decode_steps / te.last_timing.decode_seconds
        if args.shape == "360m":
            # BASELINE.json's run at this shape: batch 16, prompt lengths uniform in [64, 1024], 256 decode steps
            dec, pre, n_prompt = unequal_batch_run(te, 16, 64, 1024, 256, vocab)
            points["unequal_b16_decode"] = dec
            points["unequal_b16_prompt_tokens_per_s"] = pre
        if args.shape == "1.7b":
            # BASELINE.json's run at this shape: decode at batch 1 / 8 / 64 up to context 4096
            for b in (1, 8, 64):
                m, _, _, _, _ = decode_run(te, b, prompt_len, min(args.steps, 32), 3, vocab, context_fill=context - 64)
                points[f"decode_b{b}_ctx4096"] = b * 1000.0 / m
    line = {
        "metric": f"decode tok/s at batch 8 (SmolLM2-{args.shape.upper()} shape, prompts of 512 tokens)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"SmolLM2-{args.shape.upper()} shape, random weights", "global_batch": B, "seq_len": prompt_len, "context": context,
                   "parallelism": "single GPU", "layers": layers, "layers_of_config": full_layers,
                   "hidden": cfg["hidden_size"], "heads": H, "kv_heads": cfg["num_key_value_heads"], "head_dim": D,
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "rope_theta": cfg["rope_theta"],
                   "rms_eps": cfg["rms_norm_eps"], "tied_embeddings": True, "sampling": "greedy on device",
                   "prefill_shape": "first seen (kernels launched one by one); points.prefill_2048_replayed: from its CUDA graph",
                   "l2": "inputs larger than L2 (weights + cache > 126 MB)", "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": points,
        "clocks": clocks,
        "gpu_launches": launches,
        "library_gemm_calls": calls,
    }
    if e2e is not None:
        line["e2e"] = e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
