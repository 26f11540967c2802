"""Stand-ins for the CUDA kernels, written with plain torch on the CPU, for tests only.

They let the host-side logic (descriptors, cache bookkeeping, the step function, the generation loop)
run on a machine without a GPU, and they are the per-kernel references of the GPU kernel tests.
The product never imports this file.  `install(monkeypatch)` swaps them in.
"""
from __future__ import annotations

import torch

import plain_llama as P

PAGE = 64


def embed_gather(table, tokens, out, err=None):
    out.copy_(table[tokens.long()].float())


def add_rmsnorm(h, delta, weight, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            h += delta.float()
        src = h
    else:
        src = h[rows.long()]
        if delta is not None:
            src = src + delta[rows.long()].float()
    inv = 1.0 / torch.sqrt((src * src).sum(-1, keepdim=True) / src.shape[-1] + eps)
    out.copy_((src * inv * weight).to(out.dtype))


def residual_add(h, delta):
    h += delta.float()


def swiglu(gate_up, out):
    I = out.shape[1]
    g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_(((1.0 / (1.0 + torch.exp(-g)) * g) * u).to(out.dtype))


def convert(src, out):
    out.copy_(src.to(out.dtype))


def rope_kv_write(qkv, positions, seq_of_token, block_table, inv_freq, rot_dim, k_pages, v_pages, H, Hkv, D, err=None):
    T = qkv.shape[0]
    x = qkv.view(T, H + 2 * Hkv, D).float()
    n_rot = H + Hkv
    if rot_dim:
        half = rot_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[:, :n_rot, :half].clone(), x[:, :n_rot, half:rot_dim].clone()
        x[:, :n_rot, :half] = a * c - b * s
        x[:, :n_rot, half:rot_dim] = b * c + a * s
    qkv.view(T, H + 2 * Hkv, D)[:, :H] = x[:, :H].to(qkv.dtype)
    if k_pages is None:
        return
    for t in range(T):
        pos, seq = int(positions[t]), int(seq_of_token[t])
        page = int(block_table[seq, pos // PAGE])
        assert page >= 0
        k_pages[page, :, pos % PAGE, :] = x[t, H:H + Hkv].to(k_pages.dtype)
        v_pages[page, :, pos % PAGE, :] = x[t, H + Hkv:].to(v_pages.dtype)


def gather_kv(pages, block_table, seq, lo, hi):
    """[hi-lo+1, Hkv, D] rows of positions lo..hi of sequence `seq`."""
    rows = []
    for p in range(lo, hi + 1):
        page = int(block_table[seq, p // PAGE])
        assert page >= 0, f"position {p} of sequence {seq} has no page"
        rows.append(pages[page, :, p % PAGE, :])
    return torch.stack(rows, 0).float()


def attention_generic(q, q_row_stride, k_pages, v_pages, block_table, positions, seq_of_token, out, H, Hkv, D, scale,
                      window=0, err=None):
    T = out.shape[0]
    G = H // Hkv
    qv = q.reshape(T, -1)[:, :H * D].view(T, H, D).float()
    for t in range(T):
        pos, seq = int(positions[t]), int(seq_of_token[t])
        lo = max(0, pos - window + 1) if window else 0
        k = gather_kv(k_pages, block_table, seq, lo, pos)
        v = gather_kv(v_pages, block_table, seq, lo, pos)
        for h in range(H):
            s = (k[:, h // G, :] @ (qv[t, h] * scale))
            p = torch.softmax(s, 0)
            out[t, h * D:(h + 1) * D] = (p @ v[:, h // G, :]).to(out.dtype)


def attention(ctx, q, q_row_stride, k_pages, v_pages, block_table, out, H, Hkv, D, scale, window=0):
    attention_generic(q, q_row_stride, k_pages, v_pages, block_table, ctx.positions, ctx.seq_of_token, out, H, Hkv, D,
                      scale, window, ctx.err)


def linear(x, weight, out):
    out.copy_((x.float() @ weight.float().t()).to(out.dtype))


def sample(logits, temperature, top_p, seed, stream_id, step, out, step_add=0):
    for r in range(logits.shape[0]):
        u = P.uniform01(int(seed[r]), int(stream_id[r]), int(step[r]) + int(step_add))
        out[r] = P.sample_top_p(logits[r].numpy(), float(temperature[r]), float(top_p[r]), u)


def decode_advance(sampled, tokens, positions, ctx_len, draw_step, history, iteration):
    B = sampled.shape[0]
    it = int(iteration[0])
    tokens[:B] = sampled.clamp(min=0)
    positions += 1
    ctx_len += 1
    draw_step += 1
    history[it * B:(it + 1) * B] = sampled
    iteration += 1


def require_cuda(device):
    return torch.device("cpu")


NAMES = ["embed_gather", "add_rmsnorm", "residual_add", "swiglu", "convert", "rope_kv_write", "attention_generic",
         "attention", "linear", "sample", "decode_advance", "require_cuda"]


def install(monkeypatch):
    """Route the package's kernel calls to this file and its pinned buffers/events to plain ones."""
    from velomind_b200.engine import step
    from velomind_b200.kernels import ops
    from velomind_b200.sampling import sampler
    g = globals()
    for n in NAMES:
        monkeypatch.setattr(ops, n, g[n])

    class _Event:
        def record(self):
            pass

        def synchronize(self):
            pass

    monkeypatch.setattr(step, "GRAPHS_DEFAULT", False)
    monkeypatch.setattr(step, "_host_buffer", lambda n, dtype: torch.empty(n, dtype=dtype))
    monkeypatch.setattr(step, "_new_event", lambda: _Event())
    monkeypatch.setattr(step, "_upload", lambda dev, host, event: dev.copy_(host))
    monkeypatch.setattr(step, "_sync_stream", lambda: None)
    monkeypatch.setattr(sampler, "_host_buffer", lambda shape, dtype: torch.empty(shape, dtype=dtype))
    monkeypatch.setattr(sampler, "_sync", lambda: None)
