"""Plain torch restatements of single kernels, for the kernel tests only (the library never imports this file)."""
import torch

PAGE = 64


def rope_kv_write(qkv, positions, seq_of_token, block_table, inv_freq, rot_dim, k_pages, v_pages, H, Hkv, D, err=None, pairing=0):
    """Rotary pairs of the queries (in place) and keys; keys and values into their pages.  pairing 0: (j, j + rot_dim/2) as
    src/cpu/ops/rotary_embedding.cpp:30-44; pairing 1: (2j, 2j + 1)."""
    T = qkv.shape[0]
    x = qkv.view(T, H + 2 * Hkv, D).float()
    n_rot = H + Hkv
    if rot_dim:
        half = rot_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        ia = torch.arange(half) * 2 if pairing else torch.arange(half)
        ib = ia + 1 if pairing else ia + half
        a, b = x[:, :n_rot, ia].clone(), x[:, :n_rot, ib].clone()
        x[:, :n_rot, ia] = a * c - b * s
        x[:, :n_rot, ib] = b * c + a * s
    qkv.view(T, H + 2 * Hkv, D)[:, :H] = x[:, :H].to(qkv.dtype)
    if k_pages is None:
        return
    for t in range(T):
        pos, seq = int(positions[t]), int(seq_of_token[t])
        page = int(block_table[seq, pos // PAGE])
        assert page >= 0
        k_pages[page, :, pos % PAGE, :] = x[t, H:H + Hkv].to(k_pages.dtype)
        v_pages[page, :, pos % PAGE, :] = x[t, H + Hkv:].to(v_pages.dtype)
