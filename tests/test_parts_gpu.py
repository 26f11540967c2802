"""Each part of a layer ALONE against the plain function of the same name: the parts of a one-layer model (sizes
that no other test uses) are called one by one, outside `DecoderModel.forward`, on inputs made here, in a real step
context (descriptors, cache, workspace) of an engine.

norm, position (its frequency table), mixer (attention with its cache: a prompt step, then one token each),
feed-forward, arrangement (the block), embedding, head.
"""
import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

PARTS_CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 90, "hidden_size": 80,
    "intermediate_size": 112, "num_hidden_layers": 1, "num_attention_heads": 5, "num_key_value_heads": 1,
    "rms_norm_eps": 3e-6, "rope_theta": 5000.0, "max_position_embeddings": 512, "tie_word_embeddings": False,
    "hidden_act": "silu",
}
TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}       # times the largest reference value (at least 1)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    import velomind_b200 as vm
    d = str(tmp_path_factory.mktemp("parts_model"))
    vm.write_random_model(d, PARTS_CFG, seed=5, std=0.08, norm_jitter=0.3)
    return d


def _engine(folder, dtype):
    import velomind_b200 as vm
    model = vm.load_model(folder, dtype, DEV)
    return vm.Engine(model, 64 * 4, max_slots=2, use_graphs=False), model


class _Step:
    """A step context for `entries` with the workspace open: what a part's `forward` is given."""

    def __init__(self, engine, entries):
        self.engine, self.entries = engine, entries
        chunk = [(i, 0, len(e.tokens)) for i, e in enumerate(entries)]
        desc, T, B, R, widths, self.new_len, _ = engine._describe(entries, chunk)
        self.ctx = engine._context(desc, T, B, R, widths)
        self.ctx.run = 0

    def __enter__(self):
        self.engine.ws.begin(("parts test", self.ctx.T))
        return self.ctx

    def __exit__(self, *exc):
        self.engine.ws.end()
        torch.cuda.synchronize()
        self.engine.raise_if_error()
        for e, n in zip(self.entries, self.new_len):
            self.engine.cache.commit(e.slot, n)


def _close(got, want, dtype):
    want = np.asarray(want, dtype=np.float32)
    got = got.float().cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= TOL[dtype] * max(1.0, float(np.abs(want).max()))


def _act(x, dtype):
    """A float32 array as the activation dtype sees it (and back), so that both sides start from the same numbers."""
    t = torch.from_numpy(np.asarray(x, dtype=np.float32)).to(dtype)
    return t.to(DEV), t.float().numpy()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_embedding_head_feed_forward_alone(folder, dtype):
    import velomind_b200 as vm
    cfg, w = P.read_model(folder)
    engine, model = _engine(folder, dtype)
    rng = np.random.default_rng(1)
    hid, V = cfg["hidden_size"], cfg["vocab_size"]
    s = engine.open()
    tokens = [int(t) for t in rng.integers(0, V, 7)]
    with _Step(engine, [vm.Entry(s, tokens, [0, 6])]) as ctx:
        layer = model.layers[0]
        # ---- norm: h += delta; out = rmsnorm(h) * w
        h0 = rng.standard_normal((7, hid)).astype(np.float32) * 2
        delta_d, delta = _act(rng.standard_normal((7, hid)), dtype)
        h = torch.from_numpy(h0).to(DEV)
        out = torch.empty(7, hid, dtype=dtype, device=DEV)
        layer.block.mixer_norm.forward(ctx, h, delta_d, out)
        _close(h, h0 + delta, torch.float32)
        _close(out, P.rmsnorm(h0 + delta, w["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"]), dtype)
        rows = torch.tensor([6, 2], dtype=torch.int32, device=DEV)                     # only some rows, nothing added
        out2 = torch.empty(2, hid, dtype=dtype, device=DEV)
        model.final_norm.forward(ctx, h, None, out2, rows)
        _close(out2, P.rmsnorm((h0 + delta)[[6, 2]], w["model.norm.weight"], cfg["rms_norm_eps"]), dtype)
        # ---- embedding
        e = torch.empty(7, hid, dtype=torch.float32, device=DEV)
        model.embedding.forward(ctx, ctx.tokens, e)
        _close(e, P.embedding(w["model.embed_tokens.weight"], tokens), torch.float32)
        # ---- head (its own matrix: the embeddings are not tied here)
        x_d, x = _act(rng.standard_normal((2, hid)), dtype)
        logits = torch.empty(2, V, dtype=torch.float32, device=DEV)
        model.head.forward(ctx, x_d, logits)
        _close(logits, P.linear(x, w["lm_head.weight"]), dtype)
        # ---- feed-forward
        x_d, x = _act(rng.standard_normal((7, hid)), dtype)
        y = torch.empty(7, hid, dtype=dtype, device=DEV)
        layer.feed_forward.forward(ctx, x_d, y)
        p = "model.layers.0.mlp."
        _close(y, P.linear(P.swiglu(P.linear(x, w[p + "gate_proj.weight"]), P.linear(x, w[p + "up_proj.weight"])),
                           w[p + "down_proj.weight"]), dtype)
    engine.close(s)


def test_position_alone(folder):
    """The position part owns the frequencies: the table it hands to the mixer against the plain cosines and sines."""
    from velomind_b200.parts import PartSpec, build_part
    from velomind_b200.parts.base import BindContext
    D, theta = 48, 777.0
    part = build_part("position", PartSpec("rotary_half_split", {"head_dim": D, "theta": theta}))
    inv_freq, rot = part.tables(BindContext(torch.float32, torch.device(DEV)))
    assert rot == D and tuple(inv_freq.shape) == (D // 2,)
    positions = np.array([0, 1, 63, 64, 500], dtype=np.int32)
    cos, sin = P.rope_tables(positions, D, theta)
    angle = positions[:, None].astype(np.float32) * inv_freq.cpu().numpy()[None, :]
    assert cos.shape == angle.shape
    assert np.abs(np.cos(angle) - cos).max() < 1e-6 and np.abs(np.sin(angle) - sin).max() < 1e-6
    none = build_part("position", PartSpec("none", {}))
    assert none.tables(BindContext(torch.float32, torch.device(DEV))) == (None, 0)


def _plain_mixer(cfg, w, x, positions):
    H, Hkv, D = P.sizes(cfg)
    p = "model.layers.0.self_attn."
    S = x.shape[0]
    q = P.linear(x, w[p + "q_proj.weight"]).reshape(S, H, D)
    k = P.linear(x, w[p + "k_proj.weight"]).reshape(S, Hkv, D)
    v = P.linear(x, w[p + "v_proj.weight"]).reshape(S, Hkv, D)
    cos, sin = P.rope_tables(positions, D, cfg["rope_theta"])
    att = P.attention(P.rope(q, cos, sin), P.rope(k, cos, sin), v, 1.0 / np.sqrt(np.float32(D)), positions)
    return P.linear(att.reshape(S, H * D), w[p + "o_proj.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixer_alone_with_its_cache(folder, dtype):
    """The attention part: two prompts of unequal length in one step, then one token each from the cache the first
    step left; its inputs are made here (not the model's activations)."""
    import velomind_b200 as vm
    cfg, w = P.read_model(folder)
    engine, model = _engine(folder, dtype)
    mixer = model.layers[0].mixer
    rng = np.random.default_rng(2)
    hid = cfg["hidden_size"]
    lens = (70, 5)
    xs = [rng.standard_normal((n + 1, hid)).astype(np.float32) for n in lens]            # a prompt and one more row
    slots = [engine.open(), engine.open()]
    x_d, x = _act(np.concatenate([xs[0][:70], xs[1][:5]]), dtype)
    with _Step(engine, [vm.Entry(slots[0], [1] * 70, []), vm.Entry(slots[1], [1] * 5, [])]) as ctx:
        out = torch.empty(75, hid, dtype=dtype, device=DEV)
        mixer.forward(ctx, x_d, out)
    want = np.concatenate([_plain_mixer(cfg, w, x[:70], np.arange(70)), _plain_mixer(cfg, w, x[70:], np.arange(5))])
    _close(out, want, dtype)
    # one more token each: the keys and values of the prompts come from the cache
    y_d, y = _act(np.stack([xs[0][70], xs[1][5]]), dtype)
    with _Step(engine, [vm.Entry(slots[0], [1], [0]), vm.Entry(slots[1], [1], [0])]) as ctx:
        out = torch.empty(2, hid, dtype=dtype, device=DEV)
        mixer.forward(ctx, y_d, out)
    want = np.stack([_plain_mixer(cfg, w, np.concatenate([x[:70], y[:1]]), np.arange(71))[-1],
                     _plain_mixer(cfg, w, np.concatenate([x[70:], y[1:]]), np.arange(6))[-1]])
    _close(out, want, dtype)
    for s in slots:
        engine.close(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lens", [(9, 3), (1, 1)])
def test_arrangement_alone(folder, dtype, lens):
    """The block (norms, mixer, feed-forward and the residual sums as it wires them) on a residual stream made here:
    a step of several tokens per sequence, and a step of one token each (the fused decode kernels in bfloat16)."""
    import velomind_b200 as vm
    from velomind_b200.kernels import ops
    cfg, w = P.read_model(folder)
    engine, model = _engine(folder, dtype)
    block = model.layers[0].block
    rng = np.random.default_rng(3)
    hid = cfg["hidden_size"]
    slots = [engine.open(), engine.open()]
    h0 = rng.standard_normal((sum(lens), hid)).astype(np.float32)
    h = torch.from_numpy(h0).to(DEV)
    with _Step(engine, [vm.Entry(s, [1] * n, []) for s, n in zip(slots, lens)]) as ctx:
        pending = block.forward(ctx, h, None)
        if pending is not None:                                    # a delta the next norm would have added
            ops.residual_add(h, pending)
            ctx.ws.give(pending)
    a, b = lens
    want = np.concatenate([P.layer_forward(cfg, w, 0, h0[:a], np.arange(a)), P.layer_forward(cfg, w, 0, h0[a:], np.arange(b))])
    _close(h, want, dtype)
    for s in slots:
        engine.close(s)
