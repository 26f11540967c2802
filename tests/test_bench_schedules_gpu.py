"""The schedules that the benchmark runs, against the plain implementation: batches of 8, 24 and 64 requests of unequal
lengths that start together (the weight-streaming kernels up to 32 rows, the library products above), queued decode runs,
contexts of thousands of cached tokens up to the model's limit, prompt steps replayed from their CUDA graph, the whole
30-layer 135M shape in float32, a float32-stored model computed in bfloat16 with a shrinking batch."""
import numpy as np
import pytest

import plain_llama as P
import schedules as S
from tiny_configs import TINY_A, TINY_A_INIT, TINY_C

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2e-2}
TAILS = (3, 11, 6, 1, 8, 2, 12, 5, 9, 4)


@pytest.fixture(scope="module")
def wide_folder(tmp_path_factory):
    """SmolLM2-135M's layer sizes with four layers: the kernels run at the sizes the benchmark runs them at."""
    import velomind_b200 as vm
    cfg = dict(vm.SMOLLM2_135M, num_hidden_layers=4)
    return vm.write_random_model(str(tmp_path_factory.mktemp("wide") / "m"), cfg, seed=5, std=0.03, norm_jitter=0.2)


def _engine(folder, dtype, **kw):
    import velomind_b200 as vm
    return vm.Engine(vm.load_model(folder, dtype, "cuda:0"), **kw)


def _worst(got, want):
    scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    assert set(got) == set(want)
    return max(float(np.abs(got[k] - want[k]).max()) for k in want) / scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [8, 24, 64])
def test_batches_of_the_benchmark_match_plain(model_folders, dtype, batch):
    """`batch` requests of unequal lengths start together, the shorter ones end earlier, then a second batch takes the freed
    slots and pages: the logits of every decode step against the plain model (tiny C: the production head layout)."""
    folder = model_folders["tiny_c"]
    rng = np.random.default_rng(batch)
    lengths = [int(n) for n in rng.integers(14, 150, 2 * batch)]
    requests = S.make_requests(TINY_C["vocab_size"], lengths, seed=batch)
    plain = S.plain_logits(folder, requests)
    steps = S.steps_unequal_batches(requests, batch=batch, tails=TAILS)
    engine = _engine(folder, dtype, max_tokens=64 * 3 * batch, max_slots=batch)
    got = S.run_steps_in_process(engine, steps)
    assert _worst(got, S.expected_rows(steps, requests, plain)) <= TOL[dtype]
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0
    assert engine.graphs_captured > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("batch", [8, 64])
def test_batches_at_production_widths_match_plain(wide_folder, dtype, batch):
    rng = np.random.default_rng(100 + batch)
    lengths = [int(n) for n in rng.integers(14, 60, batch)]
    requests = S.make_requests(49152, lengths, seed=batch)
    plain = S.plain_logits(wide_folder, requests)
    steps = S.steps_unequal_batches(requests, batch=batch, tails=TAILS)
    engine = _engine(wide_folder, dtype, max_tokens=64 * 2 * batch, max_slots=batch)
    got = S.run_steps_in_process(engine, steps)
    assert _worst(got, S.expected_rows(steps, requests, plain)) <= TOL[dtype]


@pytest.mark.parametrize("batch", [8, 24, 64])
def test_queued_runs_at_the_benchmark_batches_stay_in_the_argmax_band(model_folders, batch):
    """bfloat16 greedy decoding in queued runs of 8 steps (forward, device sampler and token feedback without the host): every
    token must be, within bf16's error, a maximum of the plain model's logits at its place.  Also reports how often the token
    IS the plain model's argmax."""
    import velomind_b200 as vm
    folder = model_folders["tiny_c"]
    cfg, w = P.read_model(folder)
    rng = np.random.default_rng(7 + batch)
    prompts = [[int(t) for t in rng.integers(0, TINY_C["vocab_size"], int(n))] for n in rng.integers(3, 90, batch)]
    engine = _engine(folder, "bfloat16", max_tokens=64 * 3 * batch)
    loop = vm.GenerationLoop(engine, batch, steps_per_sync=8)
    out = loop.run([vm.Request(p, vm.SamplingParams(temperature=0.0, max_tokens=17), stream=i) for i, p in enumerate(prompts)])
    engine.raise_if_error()
    same = total = 0
    for p, r in zip(prompts[:16], out[:16]):                 # the plain model on sixteen of them is enough
        assert len(r.tokens) == 17
        ref = P.forward_logits(cfg, w, p + r.tokens[:-1])
        scale = max(1.0, float(np.abs(ref).max()))
        for j, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + j]
            assert row[tok] >= row.max() - 2 * TOL["bfloat16"] * scale, (j, tok, int(row.argmax()))
            same += int(tok == int(row.argmax()))
            total += 1
    print(f"bfloat16 argmax agreement at batch {batch}: {same}/{total}")
    assert same >= 0.9 * total
    assert engine.cache.slots.held_count == 0


def test_decoding_thousands_of_tokens_in(tmp_path):
    """One request decoded from 3,000 to 3,040 cached tokens (split-KV widths of 64 blocks), bfloat16 and float32."""
    import velomind_b200 as vm
    cfg = dict(TINY_C, max_position_embeddings=4096)
    folder = vm.write_random_model(str(tmp_path / "long"), cfg, seed=2, std=0.05, norm_jitter=0.3)
    requests = S.make_requests(cfg["vocab_size"], (3040,), seed=31)
    plain = S.plain_logits(folder, requests)
    toks = requests["r0"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": toks[:3000], "want": [0, 1500, 2999]}], "end": []}]
    steps += [{"step": 1 + j, "entries": [{"id": "r0", "tokens": [toks[3000 + j]], "want": [0]}], "end": ["r0"] if j == 39 else []} for j in range(40)]
    for dtype in ("float32", "bfloat16"):
        got = S.run_steps_in_process(_engine(folder, dtype, max_tokens=64 * 50), steps)
        assert _worst(got, S.expected_rows(steps, requests, plain)) <= TOL[dtype]


def test_prompts_of_thousands_of_tokens_take_the_warp_specialised_attention(tmp_path):
    """Head size 64 and block tables of 40 pages and more: the warp-specialised tensor-memory attention.  A prompt of 3,000
    tokens beside a short one, then a prompt cut into steps of 1,700 and 1,300 tokens (the second step's queries start 1,700
    keys in), then single tokens; logits at places spread over the prompts against the plain model, with a spike: the weights
    are scaled so that attention is sharp and a lost or doubled key block shows."""
    import velomind_b200 as vm
    cfg = dict(TINY_C, max_position_embeddings=4096)
    folder = vm.write_random_model(str(tmp_path / "long"), cfg, seed=4, std=0.06, norm_jitter=0.3)
    requests = S.make_requests(cfg["vocab_size"], (3003, 40, 3005), seed=37)
    plain = S.plain_logits(folder, requests)
    a, b, c = requests["r0"], requests["r1"], requests["r2"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": a[:3000], "want": [0, 63, 64, 127, 128, 1500, 2047, 2048, 2943, 2944, 2999]},
                                     {"id": "r1", "tokens": b, "want": [39]}], "end": ["r1"]}]
    steps += [{"step": len(steps) + j, "entries": [{"id": "r0", "tokens": [a[3000 + j]], "want": [0]}], "end": ["r0"] if j == 2 else []} for j in range(3)]
    steps.append({"step": len(steps), "entries": [{"id": "r2", "tokens": c[:1700], "want": [1699]}], "end": []})
    steps.append({"step": len(steps), "entries": [{"id": "r2", "tokens": c[1700:3000], "want": [0, 100, 1299]}], "end": []})
    steps += [{"step": len(steps) + j, "entries": [{"id": "r2", "tokens": [c[3000 + j]], "want": [0]}], "end": ["r2"] if j == 4 else []} for j in range(5)]
    engine = _engine(folder, "bfloat16", max_tokens=64 * 100)
    before = engine.counters["tc_attention_calls"]
    got = S.run_steps_in_process(engine, steps)
    engine.raise_if_error()
    assert engine.counters["tc_attention_calls"] >= before + 3 * cfg["num_hidden_layers"]
    want = S.expected_rows(steps, requests, plain)
    scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
    per_step = {k: round(float(np.abs(got[k] - want[k]).max()) / scale, 4) for k in want}
    assert max(per_step.values()) <= TOL["bfloat16"], per_step
    # the same steps twice more: their prompt shapes come a second and a third time, so the last run replays them from graphs
    recorded = engine.graphs_captured
    for again in range(2):
        got = S.run_steps_in_process(engine, steps)
        engine.raise_if_error()
        per_step = {k: round(float(np.abs(got[k] - want[k]).max()) / scale, 4) for k in want}
        assert max(per_step.values()) <= TOL["bfloat16"], (again, per_step)
    assert engine.graphs_captured >= recorded + 3          # the three prompt shapes
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0


def test_the_last_places_of_the_longest_context_and_the_refusal_beyond(tmp_path):
    """A sequence of 8,190 tokens goes on to 8,192, the model's limit (`max_position_embeddings`): the two last places still
    equal the plain model; one more token is refused on the host, and the sequence is untouched by the refusal."""
    import velomind_b200 as vm
    cfg = dict(TINY_A, max_position_embeddings=8192)
    folder = vm.write_random_model(str(tmp_path / "limit"), cfg, **TINY_A_INIT)
    requests = S.make_requests(cfg["vocab_size"], (8192,), seed=33)
    plain = S.plain_logits(folder, requests)["r0"]
    toks = requests["r0"]
    engine = _engine(folder, "bfloat16", max_tokens=8192 + 64)
    slot = engine.open()
    first = engine.step([vm.Entry(slot, toks[:8190], [8189])]).cpu().numpy().copy()
    a = engine.step([vm.Entry(slot, [toks[8190]], [0])]).cpu().numpy().copy()
    b = engine.step([vm.Entry(slot, [toks[8191]], [0])]).cpu().numpy().copy()
    scale = max(1.0, float(np.abs(plain).max()))
    for got, place in ((first, 8189), (a, 8190), (b, 8191)):
        assert np.abs(got[0] - plain[place]).max() <= TOL["bfloat16"] * scale
    assert engine.length(slot) == 8192
    with pytest.raises(vm.CacheError, match="the model's limit is 8192"):
        engine.step([vm.Entry(slot, [1], [0])])
    assert engine.length(slot) == 8192
    engine.close(slot)
    engine.raise_if_error()
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_prompt_shape_replayed_from_its_graph_matches_plain(model_folders, dtype):
    """A prompt step's first run records the buffer plan of its capacity bucket; from then on a shape that comes a second time is
    recorded into a CUDA graph and replayed: the same shape (two prompts of 70 and 9 tokens) with other tokens each time, every
    run against the plain model."""
    folder = model_folders["tiny_c"]
    engine = _engine(folder, dtype, max_tokens=64 * 8)
    recorded = []
    for run in range(4):
        requests = S.make_requests(TINY_C["vocab_size"], (70, 9), seed=40 + run)
        plain = S.plain_logits(folder, requests)
        steps = [{"step": 0, "entries": [{"id": rid, "tokens": t, "want": [0, len(t) - 1]} for rid, t in requests.items()], "end": list(requests)}]
        got = S.run_steps_in_process(engine, steps)
        assert _worst(got, S.expected_rows(steps, requests, plain)) <= TOL[dtype]
        recorded.append(engine.graphs_captured)
    assert recorded == [0, 0, 1, 1]        # the plan's run, the shape seen once (launched one by one), recorded and replayed, replayed


def test_the_whole_135m_shape_in_float32(tmp_path):
    """All 30 layers at the SmolLM2-135M sizes in true 32-bit, one cut of each kind on 64-token prompts."""
    import velomind_b200 as vm
    folder = vm.write_random_model(str(tmp_path / "m135"), vm.SMOLLM2_135M, seed=9, std=0.02)
    requests = S.make_requests(49152, (64, 64, 40), seed=50)
    plain = S.plain_logits(folder, requests)
    engine = _engine(folder, "float32", max_tokens=64 * 8, max_slots=3)
    for cut in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=8), S.steps_unequal_batches(requests)):
        got = S.run_steps_in_process(engine, cut)
        assert _worst(got, S.expected_rows(cut, requests, plain)) <= TOL["float32"]


def test_float32_stored_weights_under_bfloat16_with_a_shrinking_batch(tmp_path):
    """A tensor stored in 32-bit stays so: a float32-stored model computed with bfloat16 activations multiplies in float32
    (the input widened, the result narrowed).  Prompts of different lengths within one capacity bucket, then a batch that
    shrinks: every step of a bucket must ask the workspace for the same buffers."""
    import velomind_b200 as vm
    folder = vm.write_random_model(str(tmp_path / "f32"), TINY_A, seed=0, std=0.02, dtype="float32")
    requests = S.make_requests(TINY_A["vocab_size"], (20, 27, 31, 18), seed=60)
    plain = S.plain_logits(folder, requests)
    steps = S.steps_unequal_batches(requests, batch=4, tails=(6, 2, 4, 1))
    # a second round with other lengths in the same buckets (tokens 96 -> bucket 128; batch 4, 3, 2, 1)
    more = S.make_requests(TINY_A["vocab_size"], (25, 22, 30, 28), seed=61)
    engine = _engine(folder, "bfloat16", max_tokens=64 * 8, max_slots=4)
    got = S.run_steps_in_process(engine, steps)
    assert _worst(got, S.expected_rows(steps, requests, plain)) <= TOL["bfloat16"]
    steps2 = S.steps_unequal_batches(more, batch=4, tails=(1, 5, 2, 3))
    got2 = S.run_steps_in_process(engine, steps2)
    assert _worst(got2, S.expected_rows(steps2, more, S.plain_logits(folder, more))) <= TOL["bfloat16"]
    # steps that want no logits share nothing with steps that do
    slot = engine.open()
    engine.step([vm.Entry(slot, requests["r0"][:10], [])])
    out = engine.step([vm.Entry(slot, requests["r0"][10:], [9])]).cpu().numpy()
    assert np.abs(out[0] - plain["r0"][19]).max() <= TOL["bfloat16"] * max(1.0, float(np.abs(plain["r0"]).max()))
    engine.close(slot)
