"""Parts defined in the TESTS (tests/cpp/toy_parts.cu, a plug-in library built and loaded here) are registered, built
from a config.json, loaded and stepped without any change to the library: a mixer with fixed-size state of its own (a
decaying sum), a feed-forward with routing (top-1 of several experts), a position encoding with frequencies of its own,
and an architecture whose layers mix them with the built-in attention and SwiGLU.  Each is compared with a plain numpy
function written here.  They are toys that exist to exercise the interfaces; they are nobody's model."""
import numpy as np
import pytest

import plain_llama as P
import schedules as S

pytestmark = pytest.mark.gpu

TOY = {"architectures": ["ToyForCausalLM"], "vocab": 77, "width": 48, "layers": 4, "state": 20, "heads": 3, "experts": 3,
       "limit": 512, "decay": 0.9, "eps": 1e-5, "theta": 1000.0, "even_rotary": 1}


# ------------------------------------------------------------------------------------------ the toy parts, plain
def plain_decaying_sum(x, w_in, w_out, decay):
    """state <- decay * state + x W_in ; out = state W_out, from a zero state."""
    u = P.linear(x, w_in)
    st = np.zeros(w_in.shape[0], dtype=np.float32)
    out = np.empty((x.shape[0], w_out.shape[0]), dtype=np.float32)
    for t in range(x.shape[0]):
        st = np.float32(decay) * st + u[t]
        out[t] = w_out @ st
    return out


def plain_top_one_experts(x, w, prefix, experts):
    """A router (float32 logits, the first maximum wins) picks one small two-layer ReLU network per token."""
    choice = P.linear(x, w[prefix + "router.weight"]).argmax(-1)
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        e = int(choice[t])
        out[t] = w[prefix + f"experts.{e}.down.weight"] @ np.maximum(w[prefix + f"experts.{e}.up.weight"] @ x[t], 0)
    return out, choice


def plain_toy(c, w, tokens):
    n = len(tokens)
    positions = np.arange(n)
    h = P.embedding(w["toy.embed.weight"], tokens)
    hd = c["width"] // c["heads"]
    for l in range(c["layers"]):
        p = f"toy.layers.{l}."
        hn = P.rmsnorm(h, w[p + "mixer_norm.weight"], c["eps"])
        if l % 2 == 0:
            h = h + plain_decaying_sum(hn, w[p + "mixer.in.weight"], w[p + "mixer.out.weight"], c["decay"])
            hn = P.rmsnorm(h, w[p + "feed_forward_norm.weight"], c["eps"])
            q = "feed_forward."
            h = h + P.linear(P.swiglu(P.linear(hn, w[p + q + "gate_proj.weight"]), P.linear(hn, w[p + q + "up_proj.weight"])), w[p + q + "down_proj.weight"])
        else:
            q = P.linear(hn, w[p + "mixer.q_proj.weight"]).reshape(n, c["heads"], hd)
            k = P.linear(hn, w[p + "mixer.k_proj.weight"]).reshape(n, 1, hd)
            v = P.linear(hn, w[p + "mixer.v_proj.weight"]).reshape(n, 1, hd)
            if c["even_rotary"] and l == c["layers"] - 1:
                freq = np.arange(1, hd // 2 + 1, dtype=np.float32) * np.float32(0.5 / (hd // 2))
                angle = positions.astype(np.float32)[:, None] * freq[None, :]
                cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
            else:
                cos, sin = P.rope_tables(positions, hd, c["theta"])
            att = P.attention(P.rope(q, cos, sin), P.rope(k, cos, sin), v, 1.0 / np.sqrt(np.float32(hd)), positions)
            h = h + P.linear(att.reshape(n, c["width"]), w[p + "mixer.o_proj.weight"])
            hn = P.rmsnorm(h, w[p + "feed_forward_norm.weight"], c["eps"])
            h = h + plain_top_one_experts(hn, w, p + "feed_forward.", c["experts"])[0]
        h = h.astype(np.float32)
    return P.linear(P.rmsnorm(h, w["toy.norm.weight"], c["eps"]), w["toy.head.weight"])


@pytest.fixture
def toy_folder(tmp_path, toy_plugin):
    import velomind_b200 as vm
    assert b"toy_decaying_sum" in toy_plugin.toy_parts_registered()
    return vm.write_random_model(str(tmp_path / "toy"), TOY, seed=4, std=0.3, dtype="float32")


def test_toy_position_encoding_is_used(toy_folder, tmp_path):
    """The same weights with and without the toy frequencies in the last layer: a sequence's first token is rotated by
    angle 0 either way (equal logits), every later token is not (different logits)."""
    import velomind_b200 as vm
    plain_rotary = vm.write_random_model(str(tmp_path / "toy_geometric"), dict(TOY, even_rotary=0), seed=4, std=0.3, dtype="float32")
    tokens = [5, 70, 3, 12, 44, 9]
    rows = []
    for folder in (toy_folder, plain_rotary):
        engine = vm.Engine(vm.load_model(folder, "float32", "cuda:0"), 64 * 4)
        slot = engine.open()
        rows.append(engine.step([vm.Entry(slot, tokens, list(range(len(tokens))))]).cpu().numpy().copy())
    assert np.abs(rows[0][0] - rows[1][0]).max() < 1e-6
    assert all(np.abs(rows[0][t] - rows[1][t]).max() > 1e-4 for t in range(1, len(tokens)))


def test_toy_architecture_is_built_stepped_and_equals_plain(toy_folder):
    import velomind_b200 as vm
    cfg, w = P.read_model(toy_folder)
    model = vm.load_model(toy_folder, "float32", "cuda:0")
    engine = vm.Engine(model, 64 * 8, max_slots=3)
    groups = engine.cache.groups
    assert len(groups) == 1 and groups[0]["layers"] == 2           # only the attention layers hold keys and values
    requests = S.make_requests(TOY["vocab"], (40, 7, 100, 66, 3), seed=21)
    plain = {rid: plain_toy(cfg, w, toks) for rid, toks in requests.items()}
    scale = max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    # the routing really takes every expert somewhere (else the test would not see a wrong expert)
    hn = P.rmsnorm(P.embedding(w["toy.embed.weight"], list(range(TOY["vocab"]))), w["toy.layers.1.feed_forward_norm.weight"], TOY["eps"])
    assert len(set(plain_top_one_experts(hn, w, "toy.layers.1.feed_forward.", TOY["experts"])[1].tolist())) == TOY["experts"]
    # whole, and cut differently with slots and state areas used again: the state must carry over between steps and must be
    # cleared for a new sequence
    for cut in (S.steps_whole(requests), S.steps_tail_one_by_one(requests, tail=5), S.steps_unequal_batches(requests)):
        got = S.run_steps_in_process(engine, cut)
        exp = S.expected_rows(cut, requests, plain)
        worst = max(float(np.abs(got[k] - exp[k]).max()) for k in exp)
        assert worst < 5e-5 * scale, (worst, scale)
    # the state really matters: a slot used again gives the same answer as a fresh one only because opening it clears the state
    slot = engine.open()
    a = engine.step([vm.Entry(slot, requests["r1"], [6])]).cpu().numpy().copy()
    engine.close(slot)
    slot2 = engine.open()
    assert slot2 == slot
    b = engine.step([vm.Entry(slot2, requests["r1"], [6])]).cpu().numpy()
    engine.close(slot2)
    assert np.array_equal(a, b)
    assert engine.cache.slots.held_count == 0


def test_toy_steps_are_recorded_and_replayed(toy_folder):
    """The toy parts say that their steps may be recorded: decode steps of the toy model run from CUDA graphs and still
    equal the plain function."""
    import velomind_b200 as vm
    cfg, w = P.read_model(toy_folder)
    engine = vm.Engine(vm.load_model(toy_folder, "float32", "cuda:0"), 64 * 8)
    assert engine.use_graphs
    requests = S.make_requests(TOY["vocab"], (30, 9), seed=22)
    plain = {rid: plain_toy(cfg, w, toks) for rid, toks in requests.items()}
    steps = S.steps_tail_one_by_one(requests, tail=8)
    got = S.run_steps_in_process(engine, steps)
    exp = S.expected_rows(steps, requests, plain)
    assert max(float(np.abs(got[k] - exp[k]).max()) for k in exp) < 5e-5 * max(1.0, max(float(np.abs(v).max()) for v in plain.values()))
    assert engine.graphs_captured > 0


def test_toy_generation_through_the_entry_point(toy_folder):
    import velomind_b200 as vm
    cfg, w = P.read_model(toy_folder)
    te = vm.load(toy_folder, dtype="float32", max_tokens=1024)
    prompts = [[1, 2, 3], [70, 5], [9] * 10]
    out = te.generate(prompts, temperature=0.0, max_tokens=5, stop_tokens=())
    assert [len(r.tokens) for r in out] == [5, 5, 5]
    # greedy generation must agree with the plain toy model fed the tokens back by hand
    for p, r in zip(prompts, out):
        seq = list(p)
        for tok in r.tokens:
            row = plain_toy(cfg, w, seq)[-1]
            assert row[tok] >= row.max() - 1e-4, (seq, tok, int(row.argmax()))
            seq.append(tok)
