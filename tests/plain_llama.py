"""Plain, slow restatement of the reference's Llama decoder in numpy float32.

Whole sequences, no cache, one function for each part, nothing imported from
the package under test.  Every function cites the reference file it restates
(paths are relative to the reference project).  `tests/golden/` holds logits
made by the reference's own CPU code on a tiny random model; `test_plain.py`
compares this file with them, so this file does not rest on the formulas
alone.
"""
from __future__ import annotations

import json
import struct

import numpy as np

F = np.float32


# ----------------------------------------------------------------------------- model folder

def read_safetensors(path):
    """name -> float32 (or int32) numpy array.  BF16 is widened exactly, as
    examples/smollm2/model_loader.cpp:21-26 does (bits << 16)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    out = {}
    for name, d in header.items():
        if name == "__metadata__":
            continue
        b, e = d["data_offsets"]
        raw = blob[8 + n + b: 8 + n + e]
        if d["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif d["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4")
        elif d["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif d["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4")
        elif d["dtype"] == "I64":
            a = np.frombuffer(raw, dtype="<i8").astype(np.int32)
        else:
            raise ValueError(f"{name}: dtype {d['dtype']}")
        out[name] = a.reshape(d["shape"]).copy()
    return out


def read_model(folder):
    """(config dict, weights dict) of a model folder."""
    with open(f"{folder}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{folder}/model.safetensors")


def sizes(cfg):
    """examples/common/llama/llama_config.h:14-19: kv heads default to heads, head size = hidden / heads
    (a `head_dim` key, which the reference never reads, overrides it)."""
    H = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads") or H
    D = cfg.get("head_dim") or cfg["hidden_size"] // H
    return H, Hkv, D


# ----------------------------------------------------------------------------- parts

def embedding(table, tokens):
    """src/cpu/ops/embedding.cpp:27-32: row gather."""
    return table[np.asarray(tokens, dtype=np.int64)].astype(F)


def rmsnorm(x, w, eps):
    """src/cpu/ops/rmsnorm.cpp:42-59: y = x * (1/sqrt(mean(x^2) + eps)) * w, all float32."""
    x = x.astype(F)
    mean_sq = (x * x).sum(axis=-1, keepdims=True, dtype=F) / F(x.shape[-1])
    inv = F(1.0) / np.sqrt(mean_sq + F(eps), dtype=F)
    return (x * inv * w.astype(F)).astype(F)


def rope_tables(positions, head_dim, theta):
    """examples/common/llama/llama_rope_mask.cpp:13-25: inv_freq = 1/pow(theta, 2i/D) in float,
    angle = float(pos) * inv_freq, cos/sin of it."""
    i = np.arange(head_dim // 2, dtype=F)
    exponent = (F(2) * i) / F(head_dim)
    inv_freq = F(1.0) / np.power(F(theta), exponent, dtype=F)
    ang = np.asarray(positions, dtype=F)[:, None] * inv_freq[None, :]
    return np.cos(ang, dtype=F), np.sin(ang, dtype=F)


def rope(x, cos, sin):
    """src/cpu/ops/rotary_embedding.cpp:30-44: half-split pairs (j, j + D/2).  x [S, heads, D]."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1).astype(F)


def softmax_rows(x):
    """src/cpu/ops/softmax.cpp:28-47: max, exp(x - max), sum, divide."""
    m = x.max(axis=-1, keepdims=True)
    e = np.exp(x - m, dtype=F)
    return (e / e.sum(axis=-1, keepdims=True, dtype=F)).astype(F)


def attention(q, k, v, scale, positions=None, window=0):
    """examples/common/llama/llama_graph.cpp:97-103 with the mask of llama_rope_mask.cpp:28-41:
    scores = q k^T (scale folded into Wq by the reference's loader, model_loader.cpp:277; here it
    multiplies the scores), masked places get -1e9, softmax over keys, times v.  Query head h reads
    kv head h // G (src/cpu/ops/repeat_kv.cpp:51-61).  q [S,H,D], k/v [S,Hkv,D].
    `window` > 0 (not in the reference) also masks keys more than window-1 places back."""
    S, H, D = q.shape
    G = H // k.shape[1]
    pos = np.arange(S) if positions is None else np.asarray(positions)
    masked = pos[None, :] > pos[:, None]
    if window:
        masked |= pos[None, :] <= pos[:, None] - window
    out = np.empty((S, H, v.shape[-1]), dtype=F)
    for h in range(H):
        scores = (q[:, h, :] @ k[:, h // G, :].T).astype(F) * F(scale)
        scores = scores + np.where(masked, F(-1e9), F(0))
        out[:, h, :] = softmax_rows(scores) @ v[:, h // G, :]
    return out


def swiglu(gate, up):
    """examples/common/llama/llama_graph.cpp:22-28 and src/cpu/ops/sigmoid.cpp:23-26:
    (1/(1+exp(-g)) * g) * u."""
    sig = F(1.0) / (F(1.0) + np.exp(-gate, dtype=F))
    return ((sig * gate) * up).astype(F)


def linear(x, w):
    """src/cpu/ops/matmul.cpp:492-523 (float32 accumulate); checkpoint weights are [out, in]
    (examples/smollm2/model_loader.cpp:176-233 transposes them to [in, out])."""
    return (x.astype(F) @ w.astype(F).T).astype(F)


# ----------------------------------------------------------------------------- whole model

def layer_forward(cfg, w, l, h, positions):
    """One decoder layer, examples/common/llama/llama_graph.cpp:203-229 (pre-norm, residual after
    attention and after the feed-forward, build_mlp_block :122-138)."""
    H, Hkv, D = sizes(cfg)
    p = f"model.layers.{l}."
    S = h.shape[0]
    hn = rmsnorm(h, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    q = linear(hn, w[p + "self_attn.q_proj.weight"]).reshape(S, H, D)
    k = linear(hn, w[p + "self_attn.k_proj.weight"]).reshape(S, Hkv, D)
    v = linear(hn, w[p + "self_attn.v_proj.weight"]).reshape(S, Hkv, D)
    cos, sin = rope_tables(positions, D, cfg["rope_theta"])
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    ctx = attention(q, k, v, 1.0 / np.sqrt(F(D)), positions)
    h = h + linear(ctx.reshape(S, H * D), w[p + "self_attn.o_proj.weight"])
    hn2 = rmsnorm(h, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    ffn = swiglu(linear(hn2, w[p + "mlp.gate_proj.weight"]), linear(hn2, w[p + "mlp.up_proj.weight"]))
    return (h + linear(ffn, w[p + "mlp.down_proj.weight"])).astype(F)


def head_weight(cfg, w):
    """examples/smollm2/model_loader.cpp:124-158: lm_head.weight if the file has it, else the embedding when tied."""
    if "lm_head.weight" in w:
        return w["lm_head.weight"]
    if cfg.get("tie_word_embeddings", True):
        return w["model.embed_tokens.weight"]
    raise ValueError("lm_head.weight absent and tie_word_embeddings is false")


def forward_logits(cfg, w, tokens):
    """Logits [S, V] of one whole sequence, examples/common/llama/llama_graph.cpp:165-248."""
    tokens = list(tokens)
    positions = np.arange(len(tokens))
    h = embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["num_hidden_layers"]):
        h = layer_forward(cfg, w, l, h, positions)
    hn = rmsnorm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    return linear(hn, head_weight(cfg, w))


# ----------------------------------------------------------------------------- sampling

def philox4x32(counter, key, rounds=10):
    """Philox-4x32-10 (Salmon et al. 2011): counter 4 x uint32, key 2 x uint32 -> 4 x uint32.
    The reference draws from std::mt19937 (examples/smollm2/interactive_main.cpp:113); a counter-based
    generator replaces it so that a draw depends only on (seed, request, step)."""
    M0, M1 = 0xD2511F53, 0xCD9E8D57
    W0, W1 = 0x9E3779B9, 0xBB67AE85
    c = [int(x) & 0xFFFFFFFF for x in counter]
    k = [int(x) & 0xFFFFFFFF for x in key]
    for _ in range(rounds):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF,
             ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + W0) & 0xFFFFFFFF, (k[1] + W1) & 0xFFFFFFFF]
    return c


def uniform01(seed, stream, step):
    """A float32 in [0, 1): the top 24 bits of the first Philox word for counter (step, 0, stream, 0)
    (each 64-bit value split low word first) and key = the 64-bit seed."""
    word = philox4x32([step & 0xFFFFFFFF, (step >> 32) & 0xFFFFFFFF, stream & 0xFFFFFFFF, (stream >> 32) & 0xFFFFFFFF],
                      [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])[0]
    return F(word >> 8) * F(2.0 ** -24)


def sample_greedy(logits):
    """examples/common/llama/llama_engine.cpp:673-682: NaN skipped, the first maximum wins."""
    best, bv = -1, -np.inf
    for i, v in enumerate(logits):
        if np.isnan(v):
            continue
        if best == -1 or v > bv:
            best, bv = i, v
    return best


def sample_top_p(logits, temperature, top_p, u):
    """examples/common/llama/llama_engine.cpp:683-724 with the uniform number `u` in [0,1) handed in:
    greedy if temperature <= 0 or top_p <= 0; p_i = exp((x_i - max)/T) (float) normalised by a double
    sum; the nucleus is the smallest set of most probable tokens whose mass reaches top_p; r = u * mass;
    walk and stop at the first cumulative sum >= r.
    The reference walks in sorted order; here the walk goes in INDEX order over the nucleus, and tokens
    that tie with the least probable member all belong to it.  The distribution is the same."""
    logits = np.asarray(logits, dtype=F)
    if temperature <= 0 or top_p <= 0:
        return sample_greedy(logits)
    finite = np.isfinite(logits)
    if not finite.any():
        return -1
    max_v = logits[finite].max()
    inv_t = F(1.0) / F(temperature)
    keep = ~np.isnan(logits)
    p = np.where(keep, np.exp((logits - max_v) * inv_t, dtype=F), F(0))
    inv_sum = F(1.0 / p.astype(np.float64).sum())
    p = (p * inv_sum).astype(F)
    if F(top_p) >= F(1.0):
        tau = F(0)
    else:
        order = np.sort(p[keep])[::-1]
        cum = np.cumsum(order.astype(np.float64))
        cut = int(np.searchsorted(cum, np.float64(F(top_p)), side="left"))
        tau = order[cut] if cut < len(order) else F(0)
    member = keep & (p >= tau)
    mass = p[member].astype(np.float64).sum()
    r = np.float64(u) * mass
    acc = np.float64(0)
    last = -1
    for i in np.nonzero(member)[0]:
        acc += np.float64(p[i])
        last = int(i)
        if acc >= r:
            return last
    return last


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, top_p=1.0, seed=0, stream=0, stop=()):
    """examples/common/llama/llama_engine.cpp:633-653: sample after the prompt, then feed each token
    back; a stop token is kept in the output and ends the sequence before it is fed."""
    tokens = list(prompt)
    out = []
    for step in range(max_new_tokens):
        logits = forward_logits(cfg, w, tokens)[-1]
        nxt = sample_top_p(logits, temperature, top_p, uniform01(seed, stream, step))
        out.append(nxt)
        if nxt in stop:
            break
        tokens.append(nxt)
    return out
