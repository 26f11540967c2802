"""The engine against the plain implementation on a GPU: every way of cutting requests into steps, in
float32 and in bfloat16, on the two tiny configurations."""
import numpy as np
import pytest
import torch

import plain_llama as P
import schedules as S
from tiny_configs import TINY_A, TINY_B, TINY_C

pytestmark = pytest.mark.gpu

# float32: the reference's own bound between its cached and stateless paths is 1e-4 on the CPU and 1e-3 on
# CUDA (tests/test_smollm2_e2e.cpp:306,338; tests/test_interactive.cpp:337,354); logits here are ~1.
# bfloat16: relative to the largest logit of the run (bf16 keeps 8 bits; measured about 1 % after two or three layers).
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENGTHS = (5, 9, 2, 70, 130, 64, 65, 200, 33, 1)
CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C}


def _engine(folder, dtype, max_tokens=2048, **kw):
    import velomind_b200 as vm
    model = vm.load_model(folder, {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype], "cuda:0")
    return vm.Engine(model, max_tokens, **kw)


def _compare(got, want, tol):
    assert set(got) == set(want)
    worst = 0.0
    scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    for step in want:
        assert got[step].shape == want[step].shape, step
        assert np.isfinite(got[step]).all(), step
        worst = max(worst, float(np.abs(got[step] - want[step]).max()))
    assert worst <= tol * scale, f"max |logit - plain| = {worst:.3e} > {tol} x {scale:.2f}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("cut", ["whole", "tail", "batches", "sparse"])
def test_cuts_match_plain(model_folders, name, dtype, cut):
    folder = model_folders[name]
    requests = S.make_requests(CONFIGS[name]["vocab_size"], LENGTHS, seed=3)
    plain = S.plain_logits(folder, requests)
    steps = {"whole": S.steps_whole, "tail": S.steps_tail_one_by_one, "batches": S.steps_unequal_batches,
             "sparse": S.steps_sparse_wants}[cut](requests)
    # a cache just large enough for one batch, so that pages and slots are used again and again
    engine = _engine(folder, dtype, max_tokens=64 * 8, max_slots=3)
    got = S.run_steps_in_process(engine, steps)
    _compare(got, S.expected_rows(steps, requests, plain), TOL[dtype])
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
@pytest.mark.parametrize("cut", ["tail", "batches"])
def test_cuts_match_plain_through_the_kernel_for_large_matrices(model_folders, name, cut):
    """Steps of up to 32 rows multiply with one of two weight-streaming kernels, chosen by the size of the weight matrix; the
    tiny models never reach the one for large matrices by themselves, so it is forced here (every product of such a step
    and the head), and the logits of every step are compared with the plain model as above."""
    from velomind_b200.kernels import ops
    folder = model_folders[name]
    requests = S.make_requests(CONFIGS[name]["vocab_size"], LENGTHS, seed=13)
    plain = S.plain_logits(folder, requests)
    steps = {"tail": S.steps_tail_one_by_one, "batches": S.steps_unequal_batches}[cut](requests)
    ops.skinny_variant(2)
    try:
        engine = _engine(folder, "bfloat16", max_tokens=64 * 8, max_slots=3)
        got = S.run_steps_in_process(engine, steps)
        engine.raise_if_error()
    finally:
        ops.skinny_variant(0)
    _compare(got, S.expected_rows(steps, requests, plain), TOL["bfloat16"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_poisoned_scratch_changes_nothing(model_folders, dtype):
    """`poison_freed`: every scratch buffer is filled with NaN the moment a part gives it back (in stream order, also
    inside the recorded graphs).  A part that gave a buffer back before launching its last reader would show here."""
    folder = model_folders["tiny_b"]
    requests = S.make_requests(TINY_B["vocab_size"], LENGTHS, seed=4)
    plain = S.plain_logits(folder, requests)
    engine = _engine(folder, dtype, max_tokens=64 * 8, max_slots=3, poison_freed=True)
    steps = S.steps_unequal_batches(requests)
    got = S.run_steps_in_process(engine, steps)
    _compare(got, S.expected_rows(steps, requests, plain), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """300 tokens one by one from a 3-token prompt: crosses several pages; compared at every position."""
    folder = model_folders["tiny_b"]
    requests = S.make_requests(TINY_B["vocab_size"], (303,), seed=5)
    plain = S.plain_logits(folder, requests)
    steps = S.steps_tail_one_by_one(requests, tail=300)
    got = S.run_steps_in_process(_engine(folder, dtype), steps)
    _compare(got, S.expected_rows(steps, requests, plain), TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(model_folders, dtype):
    """A sequence fed one token at a time from its very first token, next to one that starts whole."""
    folder = model_folders["tiny_a"]
    requests = S.make_requests(TINY_A["vocab_size"], (6, 6), seed=7)
    plain = S.plain_logits(folder, requests)
    a, b = requests["r0"], requests["r1"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:1], "want": [0]}, {"id": "r1", "tokens": b, "want": [5, 0]}], "end": ["r1"]}]
    for j in range(1, 6):
        steps.append({"step": j, "entries": [{"id": "r0", "tokens": [a[j]], "want": [0]}], "end": ["r0"] if j == 5 else []})
    got = S.run_steps_in_process(_engine(folder, dtype), steps)
    _compare(got, S.expected_rows(steps, requests, plain), TOL[dtype])


def test_padding_and_company_change_nothing(model_folders):
    """float32: a request's logits are the same alone, in a batch, and cut into pieces (beyond rounding)."""
    folder = model_folders["tiny_b"]
    requests = S.make_requests(TINY_B["vocab_size"], (90, 17, 150), seed=11)
    engine = _engine(folder, "float32")
    alone = S.run_steps_in_process(engine, S.steps_whole(requests))
    toks = requests["r0"]
    steps = [
        {"step": 0, "entries": [{"id": "r0", "tokens": toks[:50], "want": list(range(50))},
                                {"id": "r2", "tokens": requests["r2"], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "r0", "tokens": toks[50:], "want": list(range(40))},
                                {"id": "r1", "tokens": requests["r1"], "want": [16]}], "end": ["r0", "r1", "r2"]},
    ]
    got = S.run_steps_in_process(engine, steps)
    cut = np.concatenate([got[0], got[1][:40]])
    assert np.abs(cut - alone[0]).max() <= 2e-6


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_entry_point(model_folders, name):
    import velomind_b200 as vm
    folder = model_folders[name]
    cfg, w = P.read_model(folder)
    prompts = [[5, 9, 2, 77, 1], [3, 4], list(range(10, 19)), [200] * 7]
    want = [P.generate(cfg, w, p, 8) for p in prompts]
    eng = vm.load(folder, dtype="float32", max_tokens=1024)
    got = eng.generate(prompts, temperature=0.0, max_tokens=8, stop_tokens=())
    assert [r.tokens for r in got] == want
    assert all(r.finish_reason == "length" for r in got)
    # bfloat16 runs the same path; a token may differ from the plain model's where two logits are close, so every token must
    # be, within bf16's error, a maximum of the plain model's logits at its place
    eng16 = vm.load(folder, dtype="bfloat16", max_tokens=1024)
    got16 = eng16.generate(prompts, temperature=0.0, max_tokens=8, stop_tokens=())
    assert [len(r.tokens) for r in got16] == [8] * 4
    same = 0
    for p, r in zip(prompts, got16):
        ref = P.forward_logits(cfg, w, p + r.tokens[:-1])
        scale = max(1.0, float(np.abs(ref).max()))
        for j, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + j]
            assert row[tok] >= row.max() - 2 * TOL["bfloat16"] * scale, (j, tok, int(row.argmax()))
            same += int(tok == int(row.argmax()))
    print(f"bfloat16 argmax agreement ({name}): {same}/32")


def test_sampled_generation_matches_plain(model_folders):
    """Temperature 0.8 with a fixed seed: the device sampler and the plain sampler draw the same tokens."""
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    cfg, w = P.read_model(folder)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7, 6]]
    want = [P.generate(cfg, w, p, 6, temperature=0.8, top_p=1.0, seed=1234, stream=i) for i, p in enumerate(prompts)]
    want_p = [P.generate(cfg, w, p, 6, temperature=0.8, top_p=0.9, seed=99, stream=i) for i, p in enumerate(prompts)]
    eng = vm.load(folder, dtype="float32", max_tokens=1024)
    got = eng.generate(prompts, temperature=0.8, top_p=1.0, max_tokens=6, seed=1234, stop_tokens=())
    assert [r.tokens for r in got] == want
    got_p = eng.generate(prompts, temperature=0.8, top_p=0.9, max_tokens=6, seed=99, stop_tokens=())
    assert [r.tokens for r in got_p] == want_p


def test_stop_token_ends_a_sequence_early(model_folders):
    import velomind_b200 as vm
    folder = model_folders["tiny_a"]
    cfg, w = P.read_model(folder)
    prompts = [[5, 9, 2, 77, 1], [3, 4]]
    free = [P.generate(cfg, w, p, 8) for p in prompts]
    stop = free[0][2]
    want = [P.generate(cfg, w, p, 8, stop=(stop,)) for p in prompts]
    eng = vm.load(folder, dtype="float32", max_tokens=1024)
    got = eng.generate(prompts, temperature=0.0, max_tokens=8, stop_tokens=(stop,))
    assert [r.tokens for r in got] == want
    assert got[0].finish_reason == "stop" and got[0].tokens[-1] == stop
    assert eng.engine.cache.slots.held_count == 0


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c"])
def test_fused_tensor_core_prefill_matches_plain(model_folders, name):
    """bfloat16 with the tcgen05 kernels (fused epilogues) switched on for every step of more than 16 tokens.
    The tiny head sizes (16, 32) are refused by the fused qkv kernel, so the attention part falls back while the
    feed-forward of tiny A (intermediate 192) takes the fused path; both must agree with the plain model."""
    folder = model_folders[name]
    requests = S.make_requests(CONFIGS[name]["vocab_size"], (150, 70, 300, 17), seed=4)
    plain = S.plain_logits(folder, requests)
    steps = S.steps_unequal_batches(requests, batch=2)
    engine = _engine(folder, "bfloat16", max_tokens=64 * 16, fused_prefill_rows=17)
    got = S.run_steps_in_process(engine, steps)
    _compare(got, S.expected_rows(steps, requests, plain), TOL["bfloat16"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_queued_decode_runs_equal_single_steps(model_folders, dtype):
    """Decode steps queued on the GPU with the tokens fed back there give the same tokens as one step at a time:
    greedy and sampled, sequences of unequal lengths crossing page boundaries, one of them stopping inside a run."""
    import velomind_b200 as vm
    folder = model_folders["tiny_c"]
    prompts = [list(range(1, 60)), [7, 8, 9], list(range(100, 230)), [5]]
    eng = vm.load(folder, dtype=dtype, max_tokens=4096)
    for temperature, top_p in ((0.0, 1.0), (0.9, 0.95)):
        one = eng.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=40, seed=11, stop_tokens=(), steps_per_sync=1)
        stop = one[1].tokens[9]
        ref = eng.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=40, seed=11, stop_tokens=(stop,), steps_per_sync=1)
        for k in (8, 64):
            got = eng.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=40, seed=11, stop_tokens=(stop,), steps_per_sync=k)
            assert [r.tokens for r in got] == [r.tokens for r in ref]
            assert [r.finish_reason for r in got] == [r.finish_reason for r in ref]
        assert any(r.finish_reason == "stop" for r in ref)
    assert eng.engine.cache.slots.held_count == 0 and eng.engine.cache.tokens_held() == 0
    eng.engine.cache.check()


@pytest.fixture(scope="module")
def wide_folder(tmp_path_factory):
    """SmolLM2-135M's layer sizes (hidden 576, 9/3 heads of 64, intermediate 1536, vocabulary 49152, tied) with
    four layers: the kernels run at the sizes the benchmark runs them at."""
    import velomind_b200 as vm
    cfg = dict(vm.SMOLLM2_135M, num_hidden_layers=4)
    return vm.write_random_model(str(tmp_path_factory.mktemp("wide") / "m"), cfg, seed=5, std=0.03, norm_jitter=0.2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_production_widths_match_plain(wide_folder, dtype):
    requests = S.make_requests(49152, (300, 40, 129), seed=8)
    plain = S.plain_logits(wide_folder, requests)
    engine = _engine(wide_folder, dtype, max_tokens=64 * 16, max_step_tokens=256)     # the 300-token prompt is cut in two
    for cut in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=20), S.steps_unequal_batches(requests)):
        got = S.run_steps_in_process(engine, cut)
        _compare(got, S.expected_rows(cut, requests, plain), TOL[dtype])
    if dtype == "bfloat16":
        fused = _engine(wide_folder, dtype, max_tokens=64 * 16, fused_prefill_rows=17)
        cut = S.steps_unequal_batches(requests)
        _compare(S.run_steps_in_process(fused, cut), S.expected_rows(cut, requests, plain), TOL[dtype])


def test_float32_cuts_agree_bit_for_bit_in_attention_order(wide_folder):
    """float32: whole, one-by-one and batched runs of the same request differ only by the library product's
    rounding (the attention kernel's reduction order does not depend on the cut)."""
    requests = S.make_requests(49152, (150,), seed=9)
    engine = _engine(wide_folder, "float32", max_tokens=64 * 8)
    a = S.run_steps_in_process(engine, S.steps_whole(requests))[0]
    tail = S.run_steps_in_process(engine, S.steps_tail_one_by_one(requests, tail=32))
    b = np.concatenate([tail[k] for k in sorted(tail)])
    assert np.abs(a - b).max() <= 2e-6 * max(1.0, float(np.abs(a).max()))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_c"])
def test_greedy_decode_tokens_are_near_argmax_of_plain(model_folders, name):
    """bfloat16 greedy decoding in queued runs: every generated token must be (within bf16's error) a maximum of the
    plain model's logits at its place."""
    import velomind_b200 as vm
    folder = model_folders[name]
    cfg, w = P.read_model(folder)
    V = CONFIGS[name]["vocab_size"]
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, V, n)] for n in (70, 3, 129, 20, 64)]
    model = vm.load_model(folder, torch.bfloat16, "cuda:0")
    engine = vm.Engine(model, 64 * 32)
    loop = vm.GenerationLoop(engine, 16, steps_per_sync=8)
    out = loop.run([vm.Request(p, vm.SamplingParams(temperature=0.0, max_tokens=30), stream=i) for i, p in enumerate(prompts)])
    engine.raise_if_error()
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 30
        ref = P.forward_logits(cfg, w, p + r.tokens[:-1])
        scale = max(1.0, float(np.abs(ref).max()))
        for j, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + j]
            assert row[tok] >= row.max() - 2 * TOL["bfloat16"] * scale, (j, tok, int(row.argmax()))
    assert engine.cache.slots.held_count == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_step_of_a_shape_while_the_default_stream_is_busy(model_folders, dtype):
    """The engine works on a stream that does not wait for the default stream.  What it prepares at the first step of a new
    shape (the step's descriptors on the device, cleared when they are made) must be ready before the step's own copies and
    kernels run, whatever else the process has queued on the default stream: here a few milliseconds of clearing a large
    tensor are queued right before every first step of a shape, and each step's logits are compared with the plain model."""
    folder = model_folders["tiny_c"]
    requests = S.make_requests(CONFIGS["tiny_c"]["vocab_size"], (300, 57, 130), seed=71)
    plain = S.plain_logits(folder, requests)
    engine = _engine(folder, dtype, max_tokens=64 * 16)
    big = torch.empty(3 << 30, dtype=torch.uint8, device="cuda:0")
    tol = TOL[dtype]
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    slots = {rid: engine.open() for rid in requests}
    import velomind_b200 as vm
    done = {rid: 0 for rid in requests}
    # steps of shapes the engine has not seen: three prompts cut at different places, then single tokens
    for cut in ((100, 57, 30), (150, 0, 60), (49, 0, 39), (1, 0, 1)):
        entries, wants = [], []
        for rid, n in zip(requests, cut):
            if n == 0:
                continue
            a = done[rid]
            entries.append(vm.Entry(slots[rid], requests[rid][a:a + n], [0, n - 1] if n > 1 else [0]))
            wants += [(rid, a), (rid, a + n - 1)] if n > 1 else [(rid, a)]
            done[rid] = a + n
        for _ in range(6):
            big.zero_()                              # a few milliseconds of work on the default stream, still running ...
        got = engine.step(entries).float().cpu().numpy()      # ... while this step's descriptors are made, copied and used
        for row, (rid, place) in zip(got, wants):
            assert np.abs(row - plain[rid][place]).max() <= tol * scale, (cut, rid, place)
    for s in slots.values():
        engine.close(s)
    engine.raise_if_error()


def test_long_prompt_takes_the_tcgen05_attention(model_folders):
    """A prompt long enough for the tensor-memory attention kernel (head size 64, more than 1,280 keys), alone and next
    to a short one, then a few tokens one by one; logits at places spread over the prompt against the plain model."""
    folder = model_folders["tiny_c"]
    requests = S.make_requests(CONFIGS["tiny_c"]["vocab_size"], (1500, 40), seed=13)
    plain = S.plain_logits(folder, requests)
    a, b = requests["r0"], requests["r1"]
    want_a = [0, 63, 64, 127, 128, 700, 1279, 1280, 1400, 1494]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:1495], "want": want_a}, {"id": "r1", "tokens": b, "want": [39]}], "end": ["r1"]}]
    for j in range(1495, 1500):
        steps.append({"step": len(steps), "entries": [{"id": "r0", "tokens": [a[j]], "want": [0]}], "end": ["r0"] if j == 1499 else []})
    engine = _engine(folder, "bfloat16", max_tokens=2048)
    got = S.run_steps_in_process(engine, steps)
    engine.raise_if_error()
    assert engine.counters["tc_attention_calls"] > 0
    _compare(got, S.expected_rows(steps, requests, plain), TOL["bfloat16"])
