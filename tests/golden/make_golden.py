"""Makes the golden logits of tests/golden/ from the REFERENCE's own CPU code.

    python tests/golden/make_golden.py /path/to/reference

Steps: write the tiny models A and B (BF16, the only storage the reference's loader takes,
examples/smollm2/model_loader.cpp:31-34) into a temporary folder; compile anchor_driver.cpp against the
reference's sources (CPU backend only); run it on fixed token lists; store tokens and logits here.
The model folders are not stored: they are re-made from (configuration, seed) by the tests.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from tiny_configs import TINY_A, TINY_A_INIT, TINY_B, TINY_B_INIT  # noqa: E402
from velomind_b200 import write_random_model  # noqa: E402

CASES = {
    "tiny_a": (TINY_A, TINY_A_INIT, [5, 17, 3, 250, 0, 99, 41, 7, 128]),
    "tiny_b": (TINY_B, TINY_B_INIT, [300, 1, 2, 3, 319, 77, 150, 9, 42, 42, 11, 200, 6]),
}


def build_anchor(ref: str, work: str) -> str:
    with open(os.path.join(work, "velomind_core_export.h"), "w") as f:     # stands in for the CMake-generated header
        f.write("#pragma once\n#define VELOMIND_CORE_EXPORT\n#define VELOMIND_CORE_NO_EXPORT\n")
    import glob
    srcs = []
    for pat in ("src/*.cpp", "src/internal/*.cpp", "src/internal/registry/*.cpp", "src/cpu/*.cpp", "src/cpu/ops/*.cpp"):
        srcs += sorted(glob.glob(os.path.join(ref, pat)))
    srcs += [os.path.join(ref, p) for p in (
        "examples/common/llama/llama_graph.cpp", "examples/common/llama/llama_rope_mask.cpp",
        "examples/smollm2/config_parser.cpp", "examples/smollm2/model_loader.cpp")]
    exe = os.path.join(work, "anchor")
    cmd = ["g++", "-std=c++23", "-O1", "-mavx2", "-mfma", "-include", "limits", f"-I{work}", f"-I{ref}/include",
           f"-I{ref}/src", f"-I{ref}/examples/common/llama", f"-I{ref}/examples/smollm2", *srcs,
           os.path.join(HERE, "anchor_driver.cpp"), "-o", exe]
    subprocess.run(cmd, check=True)
    return exe


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference project>")
    ref = sys.argv[1]
    with tempfile.TemporaryDirectory() as work:
        exe = build_anchor(ref, work)
        for name, (cfg, init, tokens) in CASES.items():
            folder = write_random_model(os.path.join(work, name), cfg, **init)
            tok_file = os.path.join(work, name + ".txt")
            with open(tok_file, "w") as f:
                f.write(" ".join(map(str, tokens)))
            out = os.path.join(work, name + ".f32")
            subprocess.run([exe, folder, tok_file, out], check=True)
            logits = np.fromfile(out, dtype="<f4").reshape(len(tokens), cfg["vocab_size"])
            np.save(os.path.join(HERE, name + "_logits.npy"), logits)
            with open(os.path.join(HERE, name + "_tokens.json"), "w") as f:
                json.dump({"tokens": tokens, "config": cfg, "init": init}, f)
            print(name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
