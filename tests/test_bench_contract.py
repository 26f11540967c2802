"""bench.py's answers that need no GPU: the reference arm's `unavailable` line, the refusal of more than one GPU, and
the roofline arithmetic (bytes of a decode step, FLOPs per token) for a known configuration."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=300,
                          env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))


def test_reference_arm_says_why_it_is_unavailable():
    """Without a CUDA device the reference arm (the reference's own benchmark tool, built from its unmodified sources)
    has no numbers: it says so in one line and exits 0."""
    proc = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


def test_reference_report_rows_are_read():
    """The reference tool's report (benchmarks/benchmark_reporter.cpp) as bench.py reads it: backend, S, graph, allocation,
    prompt ms, prompt tokens/s, decode ms, decode tokens/s."""
    sys.path.insert(0, ROOT)
    import bench
    report = (
        "| 后端 | S | 构图(中位/P95) | 分配(中位/P95) | Prefill(中位/P95) | Prefill吞吐 | Decode(中位/P95) | Decode吞吐 | D2H(中位) |\n"
        "| :--- | :---: | :---: | :---: | :---: | :---: | :---: | :---: | :---: |\n"
        "| CPU | 512 | 0.3/0.4 ms | 3.3/3.4 ms | 180.3/181.0 ms | 44.4 tok/s | 58.38/58.67 ms | 17.1 tok/s | 0.02 ms |\n"
        "| CUDA | 512 | 0.3/0.7 ms | 7.6/7.7 ms | 14.3/14.5 ms | 35741.4 tok/s | 5.74/5.80 ms | 174.3 tok/s | 0.03 ms |\n"
        "| CUDA | 2048 | 0.3/0.7 ms | 20.7/20.9 ms | 104.1/104.2 ms | 19682.6 tok/s | 12.25/12.30 ms | 81.7 tok/s | 0.03 ms |\n")
    rows = bench._parse_reference_table(report)
    assert sorted(rows) == [512, 2048]
    assert rows[512] == (14.3, 35741.4, 5.74, 174.3) and rows[2048][1] == 19682.6


def test_more_than_one_gpu_is_refused_with_one_line():
    proc = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert proc.returncode == 2
    lines = [ln for ln in proc.stdout.strip().splitlines() if ln.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0]


def test_step_bytes_and_flops_of_the_benchmark_shape():
    sys.path.insert(0, ROOT)
    import bench
    import velomind_b200 as vm
    cfg = dict(vm.SMOLLM2_135M)
    per_layer, weight_bytes, kv_per_token, D = bench.model_bytes_and_flops(cfg, cfg["num_hidden_layers"])
    hid, I, H, Hkv = 576, 1536, 9, 3
    assert D == 64
    assert per_layer == hid * (H + 2 * Hkv) * D + H * D * hid + 3 * hid * I          # weights of a layer = multiply-adds per token
    # every weight a decode step uses once, in bfloat16: the layers, the two norms' vectors and the tied table as head
    assert weight_bytes >= 2 * (30 * per_layer + cfg["vocab_size"] * hid)
    assert weight_bytes <= 2 * (30 * per_layer + cfg["vocab_size"] * hid) + 4 * 61 * hid * 2
    assert kv_per_token == 30 * 2 * Hkv * D * 2                                      # keys and values, bfloat16, per cached token
    pk = bench.peaks()
    assert pk["source"] in ("measured", "fallback") and pk["hbm_gbs"] > 0 and pk["bf16_tflops"] > 0


def test_trace_run_without_a_gpu_says_so_in_one_line(tmp_path):
    """No CPU fallback: with no CUDA device visible the replay program refuses with one clear line and exit code 1."""
    sys.path.insert(0, ROOT)
    import velomind_b200 as vm
    from tiny_configs import TINY_A, TINY_A_INIT
    folder = str(tmp_path / "model")
    vm.write_random_model(folder, TINY_A, **TINY_A_INIT)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                           "--out", str(tmp_path / "out"), "--max-tokens", "64"],
                          input='{"step": 0, "entries": [{"id": "a", "tokens": [1, 2], "want": [1]}], "end": ["a"]}\n',
                          capture_output=True, text=True, timeout=300, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert proc.returncode == 1
    lines = [ln for ln in proc.stderr.strip().splitlines() if ln.strip()]
    assert lines[-1].startswith("trace_run: error:") and "no CPU fallback" in lines[-1] and "Traceback" not in proc.stderr
    assert "done" not in proc.stdout
