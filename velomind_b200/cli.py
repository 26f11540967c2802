"""Command line in the manner of the reference's `smollm2_chat` (examples/smollm2/interactive_main.cpp:21-137):
the same option names and defaults where it has them.

    --device <cuda[:N]>   target device (the reference also takes cpu and ispc; this library has CUDA only)
    --model <path>        model folder (config.json + model.safetensors), or the path of model.safetensors
    --tokenizer <path>    tokenizer.json (default: the one in the model folder, if any)
    --synthetic           random weights at the SmolLM2-135M sizes (or --config) instead of a model folder
    --temp <float>        sampling temperature (default 0.7, 0 for greedy)
    --top-p <float>       nucleus sampling top-p (default 0.9)
    --max-tokens <int>    max generated tokens per turn (default 32)
    --prompt <string>     single non-interactive prompt; without it a `>>>` loop reads prompts
Additions: --prompt-ids 1,2,3 (token ids, for models without a tokenizer), --seed (default 42, the
reference's fixed seed), --dtype bfloat16|float32, --config <config.json> for --synthetic.
The reference's --download is not offered (no network).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

from .api import EngineConfig, TextEngine


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="smollm2_chat", description="Generate text with a Llama-architecture model on one GPU.")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--model", default="")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--config", default="", help="config.json for --synthetic (default: SmolLM2-135M sizes)")
    ap.add_argument("--temp", type=float, default=0.7)
    ap.add_argument("--top-p", type=float, default=0.9, dest="top_p")
    ap.add_argument("--max-tokens", type=int, default=32, dest="max_tokens")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--prompt-ids", default="", dest="prompt_ids")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return ap


def _device(name: str) -> str:
    if name == "cuda":
        return "cuda:0"
    if not name.startswith("cuda"):
        raise SystemExit(f"Unknown device: {name} (this library runs on cuda only; the reference's cpu and ispc backends are not built)")
    return name


def _run_turn(engine: TextEngine, prompt, args) -> None:
    print("Output: ", end="", flush=True)
    t0 = time.perf_counter()
    res = engine.generate([prompt], temperature=args.temp, top_p=args.top_p, max_tokens=args.max_tokens, seed=args.seed,
                          on_token=lambda i, tok, piece: print(piece, end="", flush=True))[0]
    dt = time.perf_counter() - t0
    rate = len(res.tokens) / dt if dt > 0 else 0.0
    print(f"\n\n[{len(res.tokens)} tokens in {dt:.3f}s ({rate:.1f} tok/s)]")


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    model_config = None
    if args.config:
        with open(args.config) as f:
            model_config = json.load(f)
    if not args.synthetic and not args.model:
        print("Error: give --model <folder> or --synthetic", file=sys.stderr)
        return 1
    try:
        cfg = EngineConfig(model_path=args.model, tokenizer_path=args.tokenizer, device=_device(args.device),
                           use_synthetic=args.synthetic, model_config=model_config, seed=args.seed, dtype=args.dtype)
        print(f"Initializing engine on device [{cfg.device}]...")
        engine = TextEngine(cfg).load()
        print("Engine ready.")
        if args.prompt_ids:
            _run_turn(engine, [int(t) for t in args.prompt_ids.replace(",", " ").split()], args)
            return 0
        if args.prompt:
            print(f"Prompt: {args.prompt}")
            # without a tokenizer the reference feeds the single token 1 (llama_engine.cpp:603-605)
            _run_turn(engine, args.prompt if engine.tokenizer is not None else [1], args)
            return 0
        while True:
            try:
                line = input(">>> ").strip()
            except EOFError:
                break
            if line in ("/exit", "/quit"):
                break
            if not line:
                continue
            if engine.tokenizer is None:
                try:
                    prompt = [int(t) for t in line.replace(",", " ").split()]
                except ValueError:
                    print("no tokenizer.json: type token ids, e.g. 1 5 17")
                    continue
            else:
                prompt = line
            _run_turn(engine, prompt, args)
    except Exception as ex:  # the reference prints "Error: <what>" and returns 1 (interactive_main.cpp:131-134)
        print(f"Error: {ex}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
