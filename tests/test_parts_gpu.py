"""Each part of a layer ALONE against the plain function of the same name.

A part is built, bound and stepped by the engine like any other, inside a probe model (tests/cpp/toy_parts.cu,
"ProbeForCausalLM") whose every other part passes the residual stream through unchanged: an identity norm, an identity
head (logits = what reaches the head) and arrangements that run only the mixer or only the feed-forward.  The token
embedding supplies the inputs (a random table: any row is as good an input as any other), at sizes no other test uses.

norm, position (through the mixer that applies it: half-split, interleaved, partial, other frequencies), mixer
(attention with its cache: a prompt step of unequal lengths, then one token each; a window), feed-forward, arrangement
(the block), embedding, head.
"""
import numpy as np
import pytest

import plain_llama as P
import schedules as S

pytestmark = pytest.mark.gpu

HID, VOCAB, HEADS, KV, D, INTER, EPS, THETA = 80, 90, 5, 1, 16, 112, 3e-6, 5000.0
TOL = {"float32": 3e-5, "bfloat16": 2e-2}       # times the largest reference value (at least 1)

IDENTITY_NORM = {"kind": "identity", "args": {"size": HID}}
RMSNORM = {"kind": "rmsnorm", "args": {"size": HID, "eps": EPS}}
IDENTITY_HEAD = {"kind": "identity", "args": {"size": HID}}
SWIGLU = {"kind": "swiglu", "args": {"hidden": HID, "intermediate": INTER}}


def _attention(position=None, window=0):
    position = position or {"kind": "rotary_half_split", "args": {"head_dim": D, "theta": THETA}}
    return {"kind": "grouped_query_attention", "args": {"hidden": HID, "heads": HEADS, "kv_heads": KV, "head_dim": D, "position": position,
                                                        "window": window}}


def _probe(vocab=HID, final_norm=IDENTITY_NORM, head=IDENTITY_HEAD, blocks=()):
    return {"architectures": ["ProbeForCausalLM"], "hidden": HID, "vocab": vocab, "limit": 512,
            "embedding": {"kind": "token_table", "args": {"vocab": vocab, "hidden": HID}}, "final_norm": final_norm, "head": head,
            "blocks": list(blocks)}


def _block(arrangement, mixer=None, feed_forward=SWIGLU, mixer_norm=IDENTITY_NORM, feed_forward_norm=IDENTITY_NORM):
    return {"arrangement": arrangement, "mixer": mixer or _attention(), "feed_forward": feed_forward, "mixer_norm": mixer_norm,
            "feed_forward_norm": feed_forward_norm}


@pytest.fixture
def build(tmp_path, toy_plugin):
    import velomind_b200 as vm

    def make(config, dtype, seed=5, std=0.5):
        folder = vm.write_random_model(str(tmp_path / f"probe{len(list(tmp_path.iterdir()))}"), config, seed=seed, std=std, norm_jitter=0.3)
        _, w = P.read_model(folder)
        model = vm.load_model(folder, dtype, "cuda:0")
        return vm.Engine(model, 64 * 6, max_slots=3), w
    return make


def _close(got, want, dtype):
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    err = float(np.abs(got - want).max())
    assert err <= TOL[dtype] * max(1.0, float(np.abs(want).max())), err


def _run(engine, steps):
    return S.run_steps_in_process(engine, steps)


def _whole(tokens_by_id):
    return [{"step": 0, "entries": [{"id": k, "tokens": v, "want": list(range(len(v)))} for k, v in tokens_by_id.items()], "end": list(tokens_by_id)}]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_norm_and_head_alone(build, dtype):
    rng = np.random.default_rng(1)
    tokens = [int(t) for t in rng.integers(0, HID, 7)]
    # ---- embedding: identity norm and head, no layer: the logits ARE the rows of the table
    engine, w = build(_probe(), dtype)
    got = _run(engine, _whole({"a": tokens}))[0]
    assert np.array_equal(got, P.embedding(w["embed.weight"], tokens))
    # ---- norm: all rows, and only some (the gather path of the last norm)
    engine, w = build(_probe(final_norm=RMSNORM), dtype)
    got = _run(engine, [{"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [6, 2]}, {"id": "b", "tokens": tokens[:3], "want": [0, 1, 2]}],
                         "end": ["a", "b"]}])[0]
    x = P.embedding(w["embed.weight"], tokens)
    _close(got, P.rmsnorm(np.concatenate([x[[6, 2]], x[:3]]), w["norm.weight"], EPS), dtype)
    # ---- head (a matrix of its own, a vocabulary that is no multiple of 8)
    tokens = [int(t) for t in rng.integers(0, VOCAB, 7)]
    engine, w = build(_probe(vocab=VOCAB, head={"kind": "linear", "args": {"vocab": VOCAB, "hidden": HID}}), dtype)
    got = _run(engine, _whole({"a": tokens}))[0]
    _close(got, P.linear(P.embedding(w["embed.weight"], tokens), w["head.weight"]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_alone(build, dtype):
    rng = np.random.default_rng(2)
    tokens = [int(t) for t in rng.integers(0, HID, 9)]
    engine, w = build(_probe(blocks=[_block("feed_forward_only")]), dtype)
    got = _run(engine, _whole({"a": tokens}))[0]
    x = P.embedding(w["embed.weight"], tokens)
    p = "layers.0.feed_forward."
    y = P.linear(P.swiglu(P.linear(x, w[p + "gate_proj.weight"]), P.linear(x, w[p + "up_proj.weight"])), w[p + "down_proj.weight"])
    _close(got - x, y, dtype)


def _rope_interleaved(x, cos, sin):
    """pairs (2j, 2j + 1) instead of the reference's (j, j + D/2); x [S, heads, R]."""
    a, b = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = a * cos[:, None, :] - b * sin[:, None, :]
    out[..., 1::2] = b * cos[:, None, :] + a * sin[:, None, :]
    return out


def _tables(positions, inv_freq):
    angle = positions.astype(np.float32)[:, None] * inv_freq[None, :].astype(np.float32)
    return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)


def _plain_mixer(w, x, positions, kind="half", rotary_dim=D, window=0, inv_freq=None):
    p = "layers.0.mixer."
    n = x.shape[0]
    q = P.linear(x, w[p + "q_proj.weight"]).reshape(n, HEADS, D)
    k = P.linear(x, w[p + "k_proj.weight"]).reshape(n, KV, D)
    v = P.linear(x, w[p + "v_proj.weight"]).reshape(n, KV, D)
    if kind != "none":
        if inv_freq is None:
            cos, sin = P.rope_tables(positions, rotary_dim, THETA)
        else:
            cos, sin = _tables(positions, inv_freq)
        turn = _rope_interleaved if kind == "interleaved" else P.rope
        q = np.concatenate([turn(q[..., :rotary_dim], cos, sin), q[..., rotary_dim:]], axis=-1)
        k = np.concatenate([turn(k[..., :rotary_dim], cos, sin), k[..., rotary_dim:]], axis=-1)
    att = P.attention(q, k, v, 1.0 / np.sqrt(np.float32(D)), positions, window=window)
    return P.linear(att.reshape(n, HEADS * D), w[p + "o_proj.weight"])


POSITIONS = {
    "half": ({"kind": "rotary_half_split", "args": {"head_dim": D, "theta": THETA}}, dict(kind="half")),
    "interleaved": ({"kind": "rotary_interleaved", "args": {"head_dim": D, "theta": THETA}}, dict(kind="interleaved")),
    "partial": ({"kind": "rotary_half_split", "args": {"head_dim": D, "theta": THETA, "rotary_dim": 8}}, dict(kind="half", rotary_dim=8)),
    "none": ({"kind": "none", "args": {}}, dict(kind="none")),
    "evenly_spaced": ({"kind": "toy_evenly_spaced_rotary", "args": {"head_dim": D, "top": 0.5, "interleaved": 0}},
                      dict(kind="half", inv_freq=np.arange(1, D // 2 + 1, dtype=np.float32) * np.float32(0.5 / (D // 2)))),
    "evenly_spaced_interleaved": ({"kind": "toy_evenly_spaced_rotary", "args": {"head_dim": D, "top": 0.5, "interleaved": 1}},
                                  dict(kind="interleaved", inv_freq=np.arange(1, D // 2 + 1, dtype=np.float32) * np.float32(0.5 / (D // 2)))),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("position", sorted(POSITIONS))
def test_mixer_alone_with_its_cache_and_every_position_encoding(build, dtype, position):
    """The attention part: two prompts of unequal length in one step, then one token each from the cache the first step left.
    The position part owns constants only; the mixer's kernels apply whatever table and pairing it hands over."""
    spec, plain_args = POSITIONS[position]
    rng = np.random.default_rng(3)
    a = [int(t) for t in rng.integers(0, HID, 71)]
    b = [int(t) for t in rng.integers(0, HID, 6)]
    engine, w = build(_probe(blocks=[_block("mixer_only", mixer=_attention(spec))]), dtype)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": list(range(70))}, {"id": "b", "tokens": b[:5], "want": list(range(5))}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:], "want": [0]}, {"id": "b", "tokens": b[5:], "want": [0]}], "end": ["a", "b"]}]
    got = _run(engine, steps)
    xa, xb = P.embedding(w["embed.weight"], a), P.embedding(w["embed.weight"], b)
    ya, yb = _plain_mixer(w, xa, np.arange(71), **plain_args), _plain_mixer(w, xb, np.arange(6), **plain_args)
    _close(got[0] - np.concatenate([xa[:70], xb[:5]]), np.concatenate([ya[:70], yb[:5]]), dtype)
    _close(got[1] - np.stack([xa[70], xb[5]]), np.stack([ya[70], yb[5]]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixer_alone_with_a_window(build, dtype):
    """A window of 70 keys: a query at position 150 must not see key 80, and the group gives pages back as the sequence grows."""
    rng = np.random.default_rng(4)
    a = [int(t) for t in rng.integers(0, HID, 160)]
    engine, w = build(_probe(blocks=[_block("mixer_only", mixer=_attention(window=70))]), dtype)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:150], "want": [0, 69, 70, 149]}], "end": []}]
    steps += [{"step": 1 + j, "entries": [{"id": "a", "tokens": [a[150 + j]], "want": [0]}], "end": ["a"] if j == 9 else []} for j in range(10)]
    got = _run(engine, steps)
    x = P.embedding(w["embed.weight"], a)
    y = _plain_mixer(w, x, np.arange(160), window=70)
    _close(got[0] - x[[0, 69, 70, 149]], y[[0, 69, 70, 149]], dtype)
    for j in range(10):
        _close(got[1 + j] - x[150 + j][None], y[150 + j][None], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lens", [(9, 3), (1, 1), (40, 1)])
def test_arrangement_alone(build, dtype, lens):
    """The block (norms, mixer, feed-forward and the residual sums as it wires them): a step of several tokens per
    sequence, and a step of one token each (the fused decode kernels in bfloat16)."""
    rng = np.random.default_rng(5)
    seqs = {f"r{i}": [int(t) for t in rng.integers(0, HID, n)] for i, n in enumerate(lens)}
    engine, w = build(_probe(blocks=[_block("prenorm", mixer_norm=RMSNORM, feed_forward_norm=RMSNORM)]), dtype, std=0.15)
    got = _run(engine, _whole(seqs))[0]
    cfg = {"hidden_size": HID, "num_attention_heads": HEADS, "num_key_value_heads": KV, "rms_norm_eps": EPS, "rope_theta": THETA,
           "intermediate_size": INTER}
    names = {"input_layernorm.": "mixer_norm.", "post_attention_layernorm.": "feed_forward_norm.", "self_attn.": "mixer.", "mlp.": "feed_forward."}
    as_llama = {}
    for k, v in w.items():
        if k.startswith("layers.0."):
            rest = k[len("layers.0."):]
            for new, old in names.items():
                if rest.startswith(old):
                    as_llama["model.layers.0." + new + rest[len(old):]] = v
    want = np.concatenate([P.layer_forward(cfg, as_llama, 0, P.embedding(w["embed.weight"], t), np.arange(len(t))) for t in seqs.values()])
    _close(got, want, dtype)
