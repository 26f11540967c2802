"""The command line end to end on a GPU: a tiny model folder, token ids in, tokens out."""
import os
import subprocess
import sys

import pytest

import plain_llama as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_smollm2_chat_single_prompt(model_folders):
    folder = model_folders["tiny_b"]
    cfg, w = P.read_model(folder)
    want = P.generate(cfg, w, [5, 6, 7, 8], 5, stop=(7, 9))
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", folder, "--dtype", "float32",
                           "--temp", "0", "--max-tokens", "5", "--prompt-ids", "5,6,7,8"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "Engine ready." in proc.stdout
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("Output: ")][0]
    assert line == "Output: " + "".join(f"[{t}]" for t in want)
    assert f"[{len(want)} tokens in" in proc.stdout
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", "/nonexistent", "--prompt-ids", "1"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "Error:" in bad.stderr
