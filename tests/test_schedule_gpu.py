"""The order in which layers run is data: a schedule that runs a layer twice (each run with a cache of its own) and
lets a run read another run's cache, registered by the tests' plug-in (tests/cpp/toy_parts.cu) as an architecture of its
own, stepped under every cut and compared with a plain whole-sequence computation that is written here from the plain
parts."""

import numpy as np
import pytest

import plain_llama as P
import schedules as S
from tiny_configs import TINY_B, TINY_B_INIT, TINY_C, TINY_C_INIT

pytestmark = pytest.mark.gpu

# (layer, run whose cache is read or None): layer 0, layer 1, layer 0 again, layer 1 again reading run 1's keys and values
SCHEDULE = ((0, None), (1, None), (0, None), (1, 1))


def _plain_looped(cfg, w, tokens):
    """Whole-sequence logits under SCHEDULE: a run that reads another run's cache projects its own queries and
    attends over the keys and values that the other run computed from ITS input."""
    H, Hkv, D = P.sizes(cfg)
    S_ = len(tokens)
    positions = np.arange(S_)
    h = P.embedding(w["model.embed_tokens.weight"], tokens)
    cos, sin = P.rope_tables(positions, D, cfg["rope_theta"])
    kept = []
    for layer, reads in SCHEDULE:
        p = f"model.layers.{layer}."
        hn = P.rmsnorm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = P.rope(P.linear(hn, w[p + "self_attn.q_proj.weight"]).reshape(S_, H, D), cos, sin)
        if reads is None:
            k = P.rope(P.linear(hn, w[p + "self_attn.k_proj.weight"]).reshape(S_, Hkv, D), cos, sin)
            v = P.linear(hn, w[p + "self_attn.v_proj.weight"]).reshape(S_, Hkv, D)
        else:
            k, v = kept[reads]
        kept.append((k, v))
        ctx = P.attention(q, k, v, 1.0 / np.sqrt(P.F(D)), positions)
        h = h + P.linear(ctx.reshape(S_, H * D), w[p + "self_attn.o_proj.weight"])
        hn2 = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        ffn = P.swiglu(P.linear(hn2, w[p + "mlp.gate_proj.weight"]), P.linear(hn2, w[p + "mlp.up_proj.weight"]))
        h = (h + P.linear(ffn, w[p + "mlp.down_proj.weight"])).astype(P.F)
    hn = P.rmsnorm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    return P.linear(hn, P.head_weight(cfg, w))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("base,init", [(TINY_B, TINY_B_INIT), (TINY_C, TINY_C_INIT)])
def test_a_layer_runs_twice_and_a_run_reads_anothers_cache(toy_plugin, tmp_path, dtype, tol, base, init):
    import velomind_b200 as vm
    cfg_json = dict(base, architectures=["LoopedLlamaForCausalLM"], num_hidden_layers=2,
                    schedule=[[layer, -1 if reads is None else reads] for layer, reads in SCHEDULE])
    folder = vm.write_random_model(str(tmp_path / "looped"), cfg_json, **init)
    cfg, w = P.read_model(folder)
    requests = S.make_requests(cfg_json["vocab_size"], (70, 5, 130, 64, 1, 33), seed=17)
    plain = {rid: _plain_looped(cfg, w, toks) for rid, toks in requests.items()}
    model = vm.load_model(folder, dtype, "cuda:0")
    assert model.info["runs"] == 4
    engine = vm.Engine(model, 64 * 8, max_slots=3)
    assert engine.cache.groups[0]["layers"] == 3                    # three runs own keys and values, the fourth borrows
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    for cut in (S.steps_whole, S.steps_tail_one_by_one, S.steps_unequal_batches):
        steps = cut(requests)
        got = S.run_steps_in_process(engine, steps)
        want = S.expected_rows(steps, requests, plain)
        worst = max(float(np.abs(got[k] - want[k]).max()) for k in want)
        assert worst <= tol * scale, (cut.__name__, worst, scale)
    engine.raise_if_error()
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0


# ------------------------------------------------------------------------------------------ layers with different cache needs
WINDOW = 70


def _plain_windowed(cfg, w, tokens):
    """Whole-sequence logits when every odd layer sees only the last WINDOW keys."""
    positions = np.arange(len(tokens))
    H, Hkv, D = P.sizes(cfg)
    S_ = len(tokens)
    h = P.embedding(w["model.embed_tokens.weight"], tokens)
    cos, sin = P.rope_tables(positions, D, cfg["rope_theta"])
    for layer in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        hn = P.rmsnorm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q = P.rope(P.linear(hn, w[p + "self_attn.q_proj.weight"]).reshape(S_, H, D), cos, sin)
        k = P.rope(P.linear(hn, w[p + "self_attn.k_proj.weight"]).reshape(S_, Hkv, D), cos, sin)
        v = P.linear(hn, w[p + "self_attn.v_proj.weight"]).reshape(S_, Hkv, D)
        ctx = P.attention(q, k, v, 1.0 / np.sqrt(P.F(D)), positions, window=WINDOW if layer % 2 else 0)
        h = h + P.linear(ctx.reshape(S_, H * D), w[p + "self_attn.o_proj.weight"])
        hn2 = P.rmsnorm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        ffn = P.swiglu(P.linear(hn2, w[p + "mlp.gate_proj.weight"]), P.linear(hn2, w[p + "mlp.up_proj.weight"]))
        h = (h + P.linear(ffn, w[p + "mlp.down_proj.weight"])).astype(P.F)
    hn = P.rmsnorm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    return P.linear(hn, P.head_weight(cfg, w))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_layers_with_a_window_keep_their_own_pages(toy_plugin, tmp_path, dtype, tol):
    """Layers that see all keys and layers that see a window of 70 in one model: two cache groups with storage of
    their own; the windowed group gives pages back while a sequence grows; every cut agrees with the plain model."""
    import velomind_b200 as vm
    cfg_json = dict(TINY_C, architectures=["WindowedLlamaForCausalLM"], num_hidden_layers=4, window=WINDOW)
    folder = vm.write_random_model(str(tmp_path / "windowed"), cfg_json, **TINY_C_INIT)
    cfg, w = P.read_model(folder)
    requests = S.make_requests(cfg_json["vocab_size"], (300, 5, 139, 71, 70, 200), seed=19)
    plain = {rid: _plain_windowed(cfg, w, toks) for rid, toks in requests.items()}
    model = vm.load_model(folder, dtype, "cuda:0")
    engine = vm.Engine(model, 64 * 12, max_slots=3)
    kinds = sorted((g["kind"], g["layers"]) for g in engine.cache.groups)
    assert kinds == [("all", 2), ("window", 2)]
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    for cut in (S.steps_whole, S.steps_tail_one_by_one, S.steps_unequal_batches):
        steps = cut(requests)
        got = S.run_steps_in_process(engine, steps)
        want = S.expected_rows(steps, requests, plain)
        worst = max(float(np.abs(got[k] - want[k]).max()) for k in want)
        assert worst <= tol * scale, (cut.__name__, worst, scale)
    # while a long sequence is held, the windowed group holds fewer pages than the group that keeps every key
    slot = engine.open()
    engine.step([vm.Entry(slot, requests["r0"], [299])])
    held = {g["kind"]: g["pages_held"] for g in engine.cache.groups}
    assert held["all"] == 5 and held["window"] < held["all"]
    engine.close(slot)
    engine.raise_if_error()
    assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0
