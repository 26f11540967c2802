"""Parts defined HERE, in the test, are registered, built from a config.json, loaded and stepped without any
change to the package: a mixer with fixed-size state of its own (a decaying sum), a feed-forward with
routing (top-1 of several experts), a position encoding with frequencies of its own, and an architecture whose
layers mix them with the built-in attention and SwiGLU.  They are toys that exist to exercise the interfaces; they are nobody's model."""
import numpy as np
import pytest
import torch

import schedules as S

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------ the toy parts
def _define():
    from velomind_b200.cache import CacheNeed
    from velomind_b200.config import KeyReader, register_architecture
    from velomind_b200.parts import BlockSpec, ModelPlan, Part, PartSpec, ScheduleEntry, register_part
    from velomind_b200.weights import WeightSpec

    class DecayingSumMixer(Part):
        """state <- decay * state + x W_in ; out = state W_out.  The state [width] per sequence is the whole
        memory of the mixer: no keys, no values."""

        def __init__(self, hidden, width, decay):
            self.hidden, self.width, self.decay = hidden, width, decay

        def weight_specs(self):
            return {"in.weight": WeightSpec((self.width, self.hidden)), "out.weight": WeightSpec((self.hidden, self.width))}

        def bind(self, weights, bc):
            self.w_in = weights["in.weight"].to(bc.device, torch.float32)
            self.w_out = weights["out.weight"].to(bc.device, torch.float32)

        def cache_need(self):
            return CacheNeed("none", state_floats=self.width)

        def forward(self, ctx, x, out):
            state = ctx.state()                                   # [max_slots, width], zero for a new sequence
            u = x.float() @ self.w_in.t()
            cu = ctx.host_cu_tokens
            for s in range(ctx.B):
                slot = int(ctx.host_slots[s])
                st = state[slot].clone()
                for t in range(int(cu[s]), int(cu[s + 1])):       # a whole prompt in one step is a scan over its tokens
                    st = self.decay * st + u[t]
                    out[t] = (st @ self.w_out.t()).to(out.dtype)
                state[slot] = st

    class TopOneExperts(Part):
        """A router picks one of `experts` small two-layer networks per token (router logits in float32)."""

        def __init__(self, hidden, inner, experts):
            self.hidden, self.inner, self.experts = hidden, inner, experts

        def weight_specs(self):
            specs = {"router.weight": WeightSpec((self.experts, self.hidden))}
            for e in range(self.experts):
                specs[f"experts.{e}.up.weight"] = WeightSpec((self.inner, self.hidden))
                specs[f"experts.{e}.down.weight"] = WeightSpec((self.hidden, self.inner))
            return specs

        def bind(self, weights, bc):
            self.w = {k: v.to(bc.device, torch.float32) for k, v in weights.items()}

        def forward(self, ctx, x, out):
            xf = x.float()
            choice = (xf @ self.w["router.weight"].t()).argmax(-1)
            y = torch.zeros_like(xf)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hcur = torch.relu(xf[rows] @ self.w[f"experts.{e}.up.weight"].t())
                    y[rows] = hcur @ self.w[f"experts.{e}.down.weight"].t()
            out.copy_(y.to(out.dtype))

    class EvenlySpacedRotary(Part):
        """Rotary pairs whose frequencies are evenly spaced between 0 and `top` instead of geometric: a position part
        owns constants only, so another table is all there is to it."""

        graph_safe = True

        def __init__(self, head_dim, top):
            self.head_dim, self.top = head_dim, top

        def tables(self, bc):
            half = self.head_dim // 2
            return (torch.arange(1, half + 1, dtype=torch.float32) * (self.top / half)).to(bc.device), self.head_dim

    def toy_config(data, where="config.json"):
        r = KeyReader(data, where)
        return {k: r.integer(k) for k in ("vocab", "width", "layers", "state", "heads", "experts", "limit")} | {
            "decay": r.number("decay"), "eps": r.number("eps"), "theta": r.number("theta"),
            "even_rotary": r.integer("even_rotary", minimum=0)}

    def toy_plan(c):
        norm = PartSpec("rmsnorm", {"size": c["width"], "eps": c["eps"]})
        blocks = []
        for l in range(c["layers"]):
            if l % 2 == 0:      # state mixer + built-in SwiGLU
                mixer = PartSpec("toy_decaying_sum", {"hidden": c["width"], "width": c["state"], "decay": c["decay"]})
                ff = PartSpec("swiglu", {"hidden": c["width"], "intermediate": 2 * c["width"]})
            else:               # built-in attention (the last one with the toy position encoding) + routed feed-forward
                hd = c["width"] // c["heads"]
                position = PartSpec("rotary_half_split", {"head_dim": hd, "theta": c["theta"]})
                if c["even_rotary"] and l == c["layers"] - 1:
                    position = PartSpec("toy_evenly_spaced_rotary", {"head_dim": hd, "top": 0.5})
                mixer = PartSpec("grouped_query_attention", {
                    "hidden": c["width"], "heads": c["heads"], "kv_heads": 1, "head_dim": hd, "position": position})
                ff = PartSpec("toy_top_one_experts", {"hidden": c["width"], "inner": c["width"], "experts": c["experts"]})
            blocks.append(BlockSpec("prenorm", f"toy.layers.{l}.", mixer, ff, norm, norm))
        return ModelPlan(hidden_size=c["width"], vocab_size=c["vocab"],
                         embedding=PartSpec("token_table", {"vocab": c["vocab"], "hidden": c["width"]}), embedding_prefix="toy.embed.",
                         blocks=tuple(blocks), schedule=tuple(ScheduleEntry(l) for l in range(c["layers"])),
                         final_norm=norm, final_norm_prefix="toy.norm.",
                         head=PartSpec("linear", {"vocab": c["vocab"], "hidden": c["width"], "tied_to": None}), head_prefix="toy.head.",
                         max_positions=c["limit"])

    register_part("mixer", "toy_decaying_sum", DecayingSumMixer)
    register_part("feed_forward", "toy_top_one_experts", TopOneExperts)
    register_part("position", "toy_evenly_spaced_rotary", EvenlySpacedRotary)
    register_architecture("ToyForCausalLM", toy_config, toy_plan)


TOY = {"architectures": ["ToyForCausalLM"], "vocab": 77, "width": 48, "layers": 4, "state": 20, "heads": 3, "experts": 3,
       "limit": 512, "decay": 0.9, "eps": 1e-5, "theta": 1000.0, "even_rotary": 1}


@pytest.fixture
def toy_folder(tmp_path):
    from velomind_b200.config import unregister_architecture
    from velomind_b200.parts import unregister_part
    import velomind_b200 as vm
    _define()
    yield vm.write_random_model(str(tmp_path / "toy"), TOY, seed=4, std=0.3, dtype="float32")
    unregister_architecture("ToyForCausalLM")
    unregister_part("mixer", "toy_decaying_sum")
    unregister_part("feed_forward", "toy_top_one_experts")
    unregister_part("position", "toy_evenly_spaced_rotary")


def test_toy_position_encoding_is_used(toy_folder, tmp_path):
    """The same weights with and without the toy frequencies in the last layer: a sequence's first token is rotated by
    angle 0 either way (equal logits), every later token is not (different logits)."""
    import velomind_b200 as vm
    plain_rotary = vm.write_random_model(str(tmp_path / "toy_geometric"), dict(TOY, even_rotary=0), seed=4, std=0.3, dtype="float32")
    tokens = [5, 70, 3, 12, 44, 9]
    rows = []
    for folder in (toy_folder, plain_rotary):
        model = vm.load_model(folder, torch.float32, "cuda:0")
        assert type(model.layers[3].mixer.position).__name__ == ("EvenlySpacedRotary" if folder == toy_folder else "RotaryHalfSplit")
        engine = vm.Engine(model, 64 * 4)
        slot = engine.open()
        rows.append(engine.step([vm.Entry(slot, tokens, list(range(len(tokens))))]).cpu().numpy().copy())
    assert np.abs(rows[0][0] - rows[1][0]).max() < 1e-6
    assert all(np.abs(rows[0][t] - rows[1][t]).max() > 1e-4 for t in range(1, len(tokens)))


def test_toy_architecture_is_built_and_stepped(toy_folder):
    import velomind_b200 as vm
    model = vm.load_model(toy_folder, torch.float32, "cuda:0")
    names = [type(l.mixer).__name__ for l in model.layers]
    assert names == ["DecayingSumMixer", "GroupedQueryAttention"] * 2
    needs = model.cache_needs()
    assert needs[0].kind == "none" and needs[0].state_floats == 20 and needs[1].kind == "all"
    engine = vm.Engine(model, 64 * 8, max_slots=3)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].n_layers == 2       # only attention layers hold keys
    assert engine.cache.state[0].shape == (3, 20) and engine.cache.state[1] is None
    requests = S.make_requests(TOY["vocab"], (40, 7, 100, 66, 3), seed=21)
    whole = S.run_steps_in_process(engine, S.steps_whole(requests))
    want = {rid: whole[i] for i, rid in enumerate(requests)}
    assert all(np.isfinite(v).all() and np.abs(v).max() > 1e-3 for v in want.values())
    # the same requests cut differently, slots and state areas used again: the state must carry over between
    # steps and must be cleared for a new sequence
    for cut in (S.steps_tail_one_by_one(requests, tail=5), S.steps_unequal_batches(requests)):
        got = S.run_steps_in_process(engine, cut)
        exp = S.expected_rows(cut, requests, want)
        scale = max(1.0, max(float(np.abs(v).max()) for v in want.values()))
        worst = max(float(np.abs(got[k] - exp[k]).max()) for k in exp)
        assert worst < 2e-5 * scale, (worst, scale)
    # the state really matters: without clearing it a reused slot would differ
    slot = engine.open()
    a = engine.step([vm.Entry(slot, requests["r1"], [6])]).cpu().numpy().copy()
    engine.close(slot)
    slot2 = engine.open()
    assert slot2 == slot
    b = engine.step([vm.Entry(slot2, requests["r1"], [6])]).cpu().numpy()
    engine.close(slot2)
    assert np.array_equal(a, b)
    assert float(engine.cache.state[0].abs().sum()) > 0          # the closed slot's state is stale, not zero ...
    slot3 = engine.open()
    assert float(engine.cache.state[0][slot3].abs().sum()) == 0  # ... until the slot is opened again


def test_toy_generation_through_the_entry_point(toy_folder):
    import velomind_b200 as vm
    te = vm.load(toy_folder, dtype="float32", max_tokens=1024)
    prompts = [[1, 2, 3], [70, 5], [9] * 10]
    out = te.generate(prompts, temperature=0.0, max_tokens=5, stop_tokens=())
    assert [len(r.tokens) for r in out] == [5, 5, 5]
    # greedy generation must agree with feeding the tokens back by hand, one whole sequence at a time
    for p, r in zip(prompts, out):
        seq = list(p)
        for tok in r.tokens:
            assert int(te.forward_logits(seq).argmax()) == tok
            seq.append(tok)
