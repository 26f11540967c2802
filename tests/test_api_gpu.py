"""The entry points on a GPU: refusals of the step function, the text engine's single-session calls and host sampling
function, the closing piece of a stream, host-side fault injection, and the two debugging switches of the launch wrappers
(wait after every launch; device time per kind of operation)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as P
from tiny_configs import TINY_A, TINY_A_INIT, TINY_B

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_step_refusals(model_folders):
    import velomind_b200 as vm
    engine = vm.Engine(vm.load_model(model_folders["tiny_a"], "float32", "cuda:0"), 128, max_slots=2)
    s = engine.open()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.step([vm.Entry(s, [1, 256], [0])])
    with pytest.raises(ValueError, match="wanted place 2"):
        engine.step([vm.Entry(s, [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([vm.Entry(s, [1], []), vm.Entry(s, [2], [])])
    with pytest.raises(vm.CacheError, match="not open"):
        engine.step([vm.Entry(1, [1], [])])
    with pytest.raises(vm.CacheError, match="max_tokens"):
        engine.step([vm.Entry(s, [1] * 129, [])])
    assert engine.length(s) == 0
    out = engine.step([vm.Entry(s, [1, 2, 3], [2, 0])]).cpu().numpy()            # wanted places keep their order
    ref = P.forward_logits(*P.read_model(model_folders["tiny_a"]), [1, 2, 3])
    assert np.abs(out - ref[[2, 0]]).max() < 5e-6
    with pytest.raises(vm.CacheError, match="model's limit"):
        engine.step([vm.Entry(s, [1] * 600, [])])
    engine.close(s)
    with pytest.raises(vm.CacheError, match="not open"):
        engine.close(s)
    with pytest.raises(vm.KernelError, match="no CPU fallback"):
        vm.load_model(model_folders["tiny_a"], "float32", "cpu")


def test_a_step_cut_into_pieces_keeps_the_asked_order(model_folders):
    """A step that brings more tokens than `max_step_tokens` is cut into pieces; wanted places asked out of order, across
    the cut, still come back in the asked order."""
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    cfg, w = P.read_model(folder)
    rng = np.random.default_rng(3)
    a, b = [int(t) for t in rng.integers(0, 320, 90)], [int(t) for t in rng.integers(0, 320, 50)]
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 8, max_step_tokens=64)
    sa, sb = engine.open(), engine.open()
    out = engine.step([vm.Entry(sa, a, [89, 3, 70]), vm.Entry(sb, b, [49, 0])]).cpu().numpy()
    ra, rb = P.forward_logits(cfg, w, a), P.forward_logits(cfg, w, b)
    want = np.stack([ra[89], ra[3], ra[70], rb[49], rb[0]])
    assert np.abs(out - want).max() < 2e-5 * max(1.0, float(np.abs(want).max()))
    engine.close(sa), engine.close(sb)


def test_text_engine_sessions_and_host_sampling_function(model_folders):
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    cfg, w = P.read_model(folder)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7, 6]]
    te = vm.TextEngine(vm.EngineConfig(model_path=folder, dtype="float32", max_tokens=512)).load()
    got = te.generate(prompts, temperature=0.8, top_p=0.95, max_tokens=4, seed=5, stop_tokens=())
    want = [P.generate(cfg, w, p, 4, temperature=0.8, top_p=0.95, seed=5, stream=i) for i, p in enumerate(prompts)]
    assert [r.tokens for r in got] == want
    assert got[0].text == "".join(f"[{t}]" for t in want[0]) and got[0].elapsed_seconds > 0 and got[0].tokens_per_second > 0
    pieces = []
    te.generate(prompts[:1], temperature=0.0, max_tokens=2, on_token=lambda i, t, piece: pieces.append(piece))
    assert len(pieces) == 2 and all(p.startswith("[") for p in pieces)         # no tokenizer: ids in brackets
    logits = te.prefill(prompts[0][:-1])
    step = te.forward_step(prompts[0][-1])
    ref = P.forward_logits(cfg, w, prompts[0])
    assert te.session_length == 7
    assert np.abs(logits.numpy() - ref[-2]).max() < 2e-5 and np.abs(step.numpy() - ref[-1]).max() < 2e-5
    assert np.abs(te.forward_logits(prompts[0]).numpy() - ref[-1]).max() < 2e-5
    assert np.abs(te.forward_full_logits(prompts[0]).numpy() - ref).max() < 2e-5
    te.reset_session()
    assert te.session_length == 0 and te.engine.cache.slots.held_count == 0
    # the reference's own way of sampling: a host function of one row of logits (llama_engine.h:106-121)
    seen = []

    def second_best(row):
        seen.append(row.shape)
        return int(np.argsort(row)[-2])

    got = te.generate([prompts[1]], max_tokens=3, stop_tokens=(), sample_fn=second_best)[0].tokens
    want, ctx = [], list(prompts[1])
    for _ in range(3):
        want.append(int(np.argsort(P.forward_logits(cfg, w, ctx)[-1])[-2]))
        ctx.append(want[-1])
    assert got == want and seen == [(cfg["vocab_size"],)] * 3
    # forward_step with the reference's position argument: only the session's length is a valid place
    te.prefill(prompts[0][:3])
    with pytest.raises(ValueError, match="not the session's length 3"):
        te.forward_step(prompts[0][3], pos=5)
    step = te.forward_step(prompts[0][3], pos=3)
    assert np.abs(step.numpy() - P.forward_logits(cfg, w, prompts[0][:4])[-1]).max() < 2e-5
    te.reset_session()
    # an exception inside a callback comes back to the caller
    with pytest.raises(ZeroDivisionError):
        te.generate(prompts[:1], temperature=0.0, max_tokens=2, on_token=lambda i, t, piece: 1 / 0)
    assert te.engine.cache.slots.held_count == 0
    # the console's description of the model (llama_interactive_console.cpp:145-158)
    d = te.describe()
    assert d["Hidden"] == 96 and d["Layers"] == 3 and d["Heads"] == "3 (kv=1)" and d["Dtype"] == "float32"


def _byte_tokenizer_json():
    """A byte-level tokenizer whose 256 tokens are the single bytes (ids 0..255), with no merges and no special tokens."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    vocab, extra = {}, 0
    for b in range(256):
        if b in keep:
            vocab[chr(b)] = b
        else:
            vocab[chr(256 + extra)] = b
            extra += 1
    return {"model": {"vocab": vocab, "merges": []}, "added_tokens": []}


def test_a_stream_ends_with_what_the_streamer_held_back(tmp_path):
    """Random tokens of a byte-level tokenizer are random bytes: pieces hold back incomplete characters, and what is still
    held back when a sequence ends comes with token -1 (examples/common/llama/llama_engine.cpp:654-655).  All pieces of a
    sequence together are its decoded text."""
    import velomind_b200 as vm
    folder = vm.write_random_model(str(tmp_path / "m"), TINY_A, **TINY_A_INIT)
    with open(os.path.join(folder, "tokenizer.json"), "w") as f:
        json.dump(_byte_tokenizer_json(), f)
    te = vm.load(folder, dtype="float32", max_tokens=1024)
    assert te.tokenizer is not None and te.tokenizer.decode([72, 105]) == "Hi" and te.tokenizer.encode("Hi") == [72, 105]
    pieces, closing = {}, []

    def on_token(i, tok, piece):
        pieces.setdefault(i, []).append(piece)
        if tok == -1:
            closing.append(i)

    prompts = ["Hello", "été", "abc"]
    out = te.generate(prompts, temperature=1.5, top_p=1.0, max_tokens=24, seed=3, stop_tokens=(), on_token=on_token)
    for i, r in enumerate(out):
        assert "".join(pieces[i]) == r.text == te.tokenizer.decode(r.tokens)
        ends_inside = r.text.endswith("�")
        assert (i in closing) == ends_inside or not ends_inside
    assert closing, "no sequence ended inside a character: choose another seed so that the closing piece is exercised"


def test_injected_failures_leave_the_engine_usable(model_folders):
    """The N-th scratch buffer of a step is refused (host-side fault injection): the step raises, holds nothing, and can be
    run again; no page or slot is lost."""
    import velomind_b200 as vm
    folder = model_folders["tiny_a"]
    ref = P.forward_logits(*P.read_model(folder), [5, 6, 7, 8])
    engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 4, max_slots=2)
    s = engine.open()
    for n in (0, 3, 7):
        engine.ws.fail_after = n
        with pytest.raises(RuntimeError, match="injected failure"):
            engine.step([vm.Entry(s, [5, 6, 7, 8], [3])])
        assert engine.length(s) == 0                                  # nothing was committed
        engine.cache.check()
    engine.ws.fail_after = None
    out = engine.step([vm.Entry(s, [5, 6, 7, 8], [3])]).cpu().numpy()
    assert np.abs(out[0] - ref[3]).max() < 2e-5
    engine.close(s)
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0


def _chat(args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), *args], capture_output=True, text=True, timeout=600,
                          env=dict(os.environ, **(env or {})))


def test_debugging_switches_of_the_launch_wrappers(model_folders):
    """`VELOMIND_B200_SYNC=1` (the host waits after every launch; recorded graphs are off), `--op-times` (two events around
    every launch) and `VELOMIND_B200_FAIL_OP` (the named operation fails after its launch), each in a process of its own."""
    folder = model_folders["tiny_a"]
    cfg, w = P.read_model(folder)
    want = "".join(f"[{t}]" for t in P.generate(cfg, w, [1, 2, 3], 5))
    base = ["--model", folder, "--fp32", "--temp", "0", "--max-tokens", "5", "--prompt-ids", "1,2,3"]
    plain_run = _chat(base)
    assert plain_run.returncode == 0 and f"Output: {want}" in plain_run.stdout, plain_run.stdout + plain_run.stderr
    synced = _chat(base, {"VELOMIND_B200_SYNC": "1"})
    assert synced.returncode == 0 and f"Output: {want}" in synced.stdout, synced.stdout + synced.stderr
    timed = _chat(base + ["--op-times"])
    assert timed.returncode == 0 and f"Output: {want}" in timed.stdout, timed.stdout + timed.stderr
    rows = {ln.split()[0]: ln.split() for ln in timed.stdout.splitlines() if ln and ln.split()[0] in ("attention_generic", "linear", "add_rmsnorm", "total")}
    assert set(rows) == {"attention_generic", "linear", "add_rmsnorm", "total"}
    assert int(rows["attention_generic"][1]) == 2 * 5 and float(rows["total"][2]) > 0          # two layers, five steps
    failed = _chat(base, {"VELOMIND_B200_FAIL_OP": "attention_generic"})
    assert failed.returncode == 1 and "attention_generic: injected failure" in failed.stderr


def test_the_console_loop_and_its_commands(model_folders, tmp_path):
    """The `>>>` loop with the reference console's commands, driven through standard input (no tokenizer: lines are ids)."""
    folder = model_folders["tiny_a"]
    cfg, w = P.read_model(folder)
    first = "".join(f"[{t}]" for t in P.generate(cfg, w, [1, 5, 17], 3))
    saved = str(tmp_path / "conversation.txt")
    script = "\n".join(["/help", "/temp 0", "/max 3", "/top_p 0.5", "/temp nonsense", "1 5 17", "/history", "/model", "/system be brief",
                        f"/save {saved}", "/clear", f"/load {saved}", "hello", "/quit"]) + "\n"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "smollm2_chat"), "--model", folder, "--fp32"], input=script, capture_output=True,
                       text=True, timeout=600)
    out = r.stdout
    assert r.returncode == 0, out + r.stderr
    assert "Commands:" in out and "Temperature set to 0" in out and "Max new tokens set to 3" in out and "Top-P set to 0.5" in out
    assert "Invalid temperature value" in out
    assert f"Output: {first}" in out and "[3 tokens in" in out
    assert "Last response: 3 tokens" in out and "Hidden:   64" in out and "Heads:    4 (kv=2)" in out
    assert "System prompt set (8 chars)." in out and f"Saved to {saved}" in out and "Conversation cleared" in out and f"Loaded from {saved}" in out
    assert "no tokenizer.json: type token ids" in out and "Exiting..." in out
    assert open(saved).read().splitlines()[:3] == ["# velomind_b200 conversation snapshot", "SYSTEM", "be brief"]
