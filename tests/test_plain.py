"""The plain implementation against logits made by the reference's own CPU code (tests/golden/), and its
sampler against hand-made cases."""
import json
import os

import numpy as np
import pytest

import plain_llama as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_build(model_folders, name):
    meta = json.load(open(os.path.join(GOLDEN, f"{name}_tokens.json")))
    gold = np.load(os.path.join(GOLDEN, f"{name}_logits.npy"))
    cfg, w = P.read_model(model_folders[name])
    mine = P.forward_logits(cfg, w, meta["tokens"])
    assert mine.shape == gold.shape
    # the reference's CPU bound between two of its own paths is 1e-4 (tests/test_smollm2_e2e.cpp:306)
    assert np.abs(mine - gold).max() < 2e-6


def test_rope_is_identity_at_position_zero_and_keeps_norm():
    x = np.random.default_rng(0).standard_normal((3, 2, 16)).astype(np.float32)
    cos, sin = P.rope_tables([0, 5, 1000], 16, 10000.0)
    y = P.rope(x, cos, sin)
    assert np.allclose(y[0], x[0])
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)


def test_attention_window_and_far_key():
    rng = np.random.default_rng(1)
    S, H, D = 40, 2, 8
    q = rng.standard_normal((S, H, D)).astype(np.float32)
    k = rng.standard_normal((S, 1, D)).astype(np.float32)
    v = rng.standard_normal((S, 1, D)).astype(np.float32)
    k[3] = 0
    k[3, 0, 0] = 50.0          # one far key that the last query scores highest ...
    q[-1, :, :] = 0
    q[-1, :, 0] = 50.0
    full = P.attention(q, k, v, 1.0)
    assert np.allclose(full[-1, 0], v[3, 0], atol=1e-4)
    win = P.attention(q, k, v, 1.0, window=8)     # ... unless the window hides it
    assert not np.allclose(win[-1, 0], v[3, 0], atol=1e-2)
    assert np.allclose(win[:8], full[:8], atol=1e-6)   # the first `window` queries see everything either way


def test_greedy_first_maximum_and_nan():
    assert P.sample_greedy(np.array([1.0, 3.0, 3.0, np.nan], dtype=np.float32)) == 1
    assert P.sample_greedy(np.array([np.nan, np.nan], dtype=np.float32)) == -1
    assert P.sample_top_p(np.array([0.0, 2.0], dtype=np.float32), 0.0, 0.9, 0.5) == 1
    assert P.sample_top_p(np.array([0.0, 2.0], dtype=np.float32), 0.7, 0.0, 0.5) == 1


def test_top_p_cut_and_walk():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    # nucleus of 0.7: tokens 0 and 1 (mass 0.8); u walks them in index order
    assert P.sample_top_p(logits, 1.0, 0.7, 0.0) == 0
    assert P.sample_top_p(logits, 1.0, 0.7, 0.6) == 0
    assert P.sample_top_p(logits, 1.0, 0.7, 0.7) == 1
    assert P.sample_top_p(logits, 1.0, 0.7, 0.999) == 1
    # everything: the last token is reachable
    assert P.sample_top_p(logits, 1.0, 1.0, 0.999) == 3
    counts = np.zeros(4)
    for step in range(4000):
        counts[P.sample_top_p(logits, 1.0, 1.0, P.uniform01(5, 0, step))] += 1
    assert np.abs(counts / 4000 - [0.5, 0.3, 0.15, 0.05]).max() < 0.03


def test_philox_known_answer():
    # Random123 known-answer vectors for philox4x32-10
    assert P.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert P.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert P.philox4x32([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
