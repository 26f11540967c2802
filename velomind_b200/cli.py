"""Command line in the manner of the reference's `smollm2_chat` (examples/smollm2/interactive_main.cpp:21-137):
the same option names and defaults where it has them.

    --device <cuda[:N]>   target device (the reference also takes cpu and ispc; this library has CUDA only)
    --model <path>        model folder (config.json + model.safetensors), or the path of model.safetensors
    --tokenizer <path>    tokenizer.json (default: the one in the model folder, if any)
    --synthetic           random weights at the SmolLM2-135M sizes (or --config) instead of a model folder
    --temp <float>        sampling temperature (default 0.7, 0 for greedy)
    --top-p <float>       nucleus sampling top-p (default 0.9)
    --max-tokens <int>    max generated tokens per turn (default 32)
    --prompt <string>     single non-interactive prompt; without it a `>>>` loop reads prompts and the
                          reference console's commands (examples/common/llama/llama_interactive_console.cpp:125-309):
                          /help /temp /top_p /max /system /clear /history /model /save /load /exit /quit
Additions: --prompt-ids 1,2,3 (token ids, for models without a tokenizer), --prompt-file <path>, --seed (default 42,
the reference's fixed seed), --dtype bfloat16|float32 (--fp32 for short), --config <config.json> for --synthetic,
--op-times (device time per kind of operation after each response).
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
    ap.add_argument("--prompt-file", default="", dest="prompt_file",
                    help="a file holding the prompt: text, or token ids when the model has no tokenizer")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--fp32", action="store_true", help="the true 32-bit path of the whole model (the same as --dtype float32)")
    ap.add_argument("--op-times", action="store_true", dest="op_times",
                    help="after each response, print the device time per kind of operation (kernels launched one by one, no CUDA graphs)")
    return ap


def _device(name: str) -> str:
    if name == "cuda":
        return "cuda:0"
    if not name.startswith("cuda"):
        raise SystemExit(f"Unknown device: {name} (this library runs on cuda only; the reference's cpu and ispc backends are not built)")
    return name


def _run_turn(engine: TextEngine, prompt, args):
    """One response, streamed to the terminal; returns (result, seconds, the text that was printed)."""
    print("Output: ", end="", flush=True)
    pieces = []

    def show(i, tok, piece):
        pieces.append(piece)
        print(piece, end="", flush=True)

    t0 = time.perf_counter()
    if getattr(args, "op_times", False):
        from .kernels.optimes import OpTimes
        with OpTimes() as times:
            res = engine.generate([prompt], temperature=args.temp, top_p=args.top_p, max_tokens=args.max_tokens, seed=args.seed,
                                  on_token=show)[0]
        dt = time.perf_counter() - t0
        print("\n\n" + times.table(), end="")
    else:
        res = engine.generate([prompt], temperature=args.temp, top_p=args.top_p, max_tokens=args.max_tokens, seed=args.seed,
                              on_token=show)[0]
        dt = time.perf_counter() - t0
    rate = len(res.tokens) / dt if dt > 0 else 0.0
    print(f"\n\n[{len(res.tokens)} tokens in {dt:.3f}s ({rate:.1f} tok/s)]")
    return res, dt, "".join(pieces)


class Console:
    """The `>>>` loop's state and slash commands, with the meanings the reference's console gives them
    (llama_interactive_console.cpp:25-41 state, :125-143 help, :224-309 commands, :104-117 how a prompt is composed):
    the conversation is a list of turns (user, assistant, user, ...); a prompt is the system text, the turns and the new
    line joined by newlines; /clear forgets the turns and keeps the system text; every turn takes the next seed.
    Without a tokenizer a line is a list of token ids and stands alone (there is no text to join)."""

    HELP = ("  /help               Show commands + current state.",
            "  /temp <float>       Sampling temperature (0 = greedy). Current: {temp}",
            "  /top_p <float>      Nucleus top-p threshold. Current: {top_p}",
            "  /max <int>          Max generated tokens per response. Current: {max_tokens}",
            "  /system <text>      Set/replace the system prompt prefix (no text: clear it).",
            "  /clear              Clear conversation history (keeps system).",
            "  /history            Show per-turn stats for the last response.",
            "  /model              Show model info (path / config / device).",
            "  /save <file>        Persist conversation history to file.",
            "  /load <file>        Load conversation history from file.",
            "  /exit, /quit        Exit.")

    def __init__(self, engine, args, out=print):
        self.engine, self.args, self.out = engine, args, out
        self.system = ""
        self.turns = []
        self.last = (0, 0.0, "")           # tokens, seconds, text of the last response

    # ---- commands: True = handled, False = leave the loop, None = not a command (a prompt)
    def command(self, line: str):
        a = self.args
        if line in ("/exit", "/quit"):
            self.out("Exiting...")
            return False
        if line == "/help":
            self.out("Commands:")
            for h in self.HELP:
                self.out(h.format(temp=a.temp, top_p=a.top_p, max_tokens=a.max_tokens))
            self.out(f"\nModel path: {a.model}\nTokenizer:  {a.tokenizer}\nDevice:     {a.device}\n"
                     f"Synthetic:  {'yes' if a.synthetic else 'no'}\n")
            return True
        if line == "/model":
            for k, v in self.engine.describe().items():
                self.out(f"{k + ':':<10}{v}")
            self.out("")
            return True
        if line == "/history":
            n, dt, text = self.last
            self.out(f"Last response: {n} tokens in {dt:.2f}s ({(n / dt if dt > 0 else 0.0):.1f} tok/s)\nLast text: {text}\n")
            return True
        if line == "/clear":
            self.turns.clear()
            self.out("Conversation cleared (system prompt retained).\n")
            return True
        for name, attr, kind, label in (("/temp ", "temp", float, "Temperature"), ("/top_p ", "top_p", float, "Top-P"),
                                        ("/max ", "max_tokens", int, "Max new tokens")):
            if line.startswith(name):
                try:
                    value = kind(line[len(name):].strip())
                    if kind is int and value < 0:
                        raise ValueError
                    setattr(a, attr, value)
                    self.out(f"{label} set to {value}\n")
                except ValueError:
                    self.out(f"Invalid {label.lower()} value\n")
                return True
        if line == "/system" or line.startswith("/system "):
            self.system = line[len("/system "):] if line.startswith("/system ") else ""
            self.out(f"System prompt set ({len(self.system)} chars).\n" if self.system else "System prompt cleared.\n")
            return True
        if line.startswith("/save "):
            path = line[len("/save "):].strip()
            try:
                with open(path, "w") as f:
                    f.write(self.snapshot())
                self.out(f"Saved to {path}\n")
            except OSError as ex:
                self.out(f"Save failed: {ex}\n")
            return True
        if line.startswith("/load "):
            path = line[len("/load "):].strip()
            try:
                with open(path) as f:
                    self.restore(f.read())
                self.out(f"Loaded from {path} ({len(self.turns)} turns)\n")
            except OSError as ex:
                self.out(f"Load failed: {ex}\n")
            return True
        return None

    # ---- the conversation as a file: role lines (SYSTEM / USER / ASSISTANT), each followed by the text; # lines are comments
    def snapshot(self) -> str:
        parts = ["# velomind_b200 conversation snapshot"]
        if self.system:
            parts += ["SYSTEM", self.system]
        for i, t in enumerate(self.turns):
            parts += ["USER" if i % 2 == 0 else "ASSISTANT", t]
        return "\n".join(parts) + "\n"

    def restore(self, text: str) -> None:
        self.system, self.turns = "", []
        role, body = None, []

        def flush():
            if role == "SYSTEM":
                self.system = "\n".join(body)
            elif role in ("USER", "ASSISTANT"):
                self.turns.append("\n".join(body))

        for ln in text.splitlines():
            if ln.startswith("#") or ln in ("SYSTEM", "USER", "ASSISTANT"):
                flush()
                role, body = (None if ln.startswith("#") else ln), []
            else:
                body.append(ln)
        flush()

    def compose(self, user_text: str) -> str:
        return "\n".join(([self.system] if self.system else []) + self.turns + [user_text])

    def turn(self, line: str) -> None:
        if self.engine.tokenizer is None:
            try:
                prompt = [int(t) for t in line.replace(",", " ").split()]
            except ValueError:
                self.out("no tokenizer.json: type token ids, e.g. 1 5 17")
                return
        else:
            prompt = self.compose(line)
        res, dt, text = _run_turn(self.engine, prompt, self.args)
        self.args.seed += 1
        self.last = (len(res.tokens), dt, text)
        if self.engine.tokenizer is not None:
            self.turns += [line, text]


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.fp32:
        args.dtype = "float32"
    model_config = None
    if args.config:
        with open(args.config) as f:
            model_config = json.load(f)
    if not args.synthetic and not args.model:
        print("Error: give --model <folder> or --synthetic", file=sys.stderr)
        return 1
    try:
        cfg = EngineConfig(model_path=args.model, tokenizer_path=args.tokenizer, device=_device(args.device),
                           use_synthetic=args.synthetic, model_config=model_config, seed=args.seed, dtype=args.dtype,
                           use_graphs=False if args.op_times else None)
        print(f"Initializing engine on device [{cfg.device}]...")
        engine = TextEngine(cfg).load()
        print("Engine ready.")
        if args.prompt_file:
            with open(args.prompt_file) as f:
                text = f.read().strip()
            if engine.tokenizer is None:
                args.prompt_ids = text
            else:
                args.prompt = text
        if args.prompt_ids:
            _run_turn(engine, [int(t) for t in args.prompt_ids.replace(",", " ").split()], args)
            return 0
        if args.prompt:
            print(f"Prompt: {args.prompt}")
            # without a tokenizer the reference feeds the single token 1 (llama_engine.cpp:603-605)
            _run_turn(engine, args.prompt if engine.tokenizer is not None else [1], args)
            return 0
        console = Console(engine, args)
        while True:
            try:
                line = input(">>> ").strip()
            except EOFError:
                break
            if not line:
                continue
            handled = console.command(line) if line.startswith("/") else None
            if handled is False:
                break
            if handled is None:
                console.turn(line)
    except Exception as ex:  # the reference prints "Error: <what>" and returns 1 (interactive_main.cpp:131-134)
        print(f"Error: {ex}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
