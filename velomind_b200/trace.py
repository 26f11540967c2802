"""Trace replay: feed given token ids through a model step by step and write logits.  Samples nothing.

It drives the same model, step function, cache and kernels that generation uses.

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, `<out>/<step>.f32` receives the logits at the wanted places in
the order of the entries and of `want`, little-endian float32 [wanted, vocab].  After every step a line
`done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import torch

from . import models  # noqa: F401
from .engine.model import load_model
from .engine.step import Engine, Entry


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    os.makedirs(args.out, exist_ok=True)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    model = load_model(args.model, dtype, args.device)
    engine = Engine(model, args.max_tokens)
    slots: Dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.open()
            entries.append(Entry(slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                host = logits.to("cpu")          # synchronises
                host.numpy().astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
            engine.raise_if_error()
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                engine.close(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


def run(argv=None) -> int:
    """`main` for the command line: a failure is one line on stderr and exit code 1, not a traceback."""
    try:
        return main(argv)
    except (KeyboardInterrupt, BrokenPipeError):
        return 130
    except Exception as ex:
        if os.environ.get("VELOMIND_B200_TRACEBACK", "") == "1":
            raise
        print(f"trace_run: error: {type(ex).__name__}: {ex}   (VELOMIND_B200_TRACEBACK=1 shows where)", file=sys.stderr, flush=True)
        return 1


if __name__ == "__main__":
    sys.exit(run())
