"""bin/trace_run as a user runs it: a subprocess fed JSON lines, writing <step>.f32 files."""
import os
import subprocess
import sys

import numpy as np
import pytest

import schedules as S
from tiny_configs import TINY_A, TINY_B

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-5, "bfloat16": 2e-2}     # times the largest logit (at least 1)


def _replay(folder, dtype, steps, out, max_tokens):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)], input=S.to_jsonl(steps), text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", [("tiny_a", TINY_A), ("tiny_b", TINY_B)])
def test_replay_three_cuts(model_folders, tmp_path, name, cfg, dtype):
    folder = model_folders[name]
    requests = S.make_requests(cfg["vocab_size"], (40, 7, 100, 66, 35, 129), seed=13)
    plain = S.plain_logits(folder, requests)
    cuts = {"whole": S.steps_whole, "tail": S.steps_tail_one_by_one, "batches": S.steps_unequal_batches,
            "sparse": S.steps_sparse_wants}
    # one process replays all the cuts, one after another, with a cache of 8 pages: pages and slots are used again
    steps, owner, all_requests, all_plain = [], {}, {}, {}
    for cut, make in cuts.items():
        renamed = {f"{cut}:{rid}": toks for rid, toks in requests.items()}
        all_requests.update(renamed)
        all_plain.update({f"{cut}:{rid}": plain[rid] for rid in requests})
        for r in make(renamed):
            r = dict(r, step=len(steps))
            owner[r["step"]] = cut
            steps.append(r)
    out = str(tmp_path / "out")
    _replay(folder, dtype, steps, out, max_tokens=64 * 8)
    want = S.expected_rows(steps, all_requests, all_plain)
    scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    for step, rows in want.items():
        got = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, cfg["vocab_size"])
        assert got.shape == rows.shape, (step, owner[step])
        err = float(np.abs(got - rows).max())
        assert err <= TOL[dtype] * scale, f"step {step} of cut {owner[step]!r}: max |logit - plain| = {err:.3e}"
    assert sorted(int(f[:-4]) for f in os.listdir(out)) == sorted(want)
