"""Each CUDA kernel alone against a plain float32 reference, at sizes other than the engine tests use:
head sizes in steps of 16, odd head counts and groups, widths and vocabularies that are no power of two."""
import math

import numpy as np
import pytest
import torch

import kernel_refs as E
import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from velomind_b200.kernels import ops as o
    return o


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(table_dtype):
    V, hid, T = 1000, 136, 37
    table = torch.randn(V, hid, generator=_gen(0)).to(table_dtype)
    tokens = torch.randint(0, V, (T,), generator=_gen(1), dtype=torch.int32)
    out = torch.empty(T, hid, device=DEV)
    ops().embed_gather(table.to(DEV), tokens.to(DEV), out)
    assert torch.equal(out.cpu(), table[tokens.long()].float())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("hid", [200, 576, 1600, 4100])      # (1600: a row no longer fits a warp's registers)
@pytest.mark.parametrize("T", [19, 131])          # few rows: a block per row; many rows (bfloat16): a warp per row, four values per load
def test_add_rmsnorm(dtype, tol, hid, T):
    eps = 3e-6
    h = torch.randn(T, hid, generator=_gen(2)) * 3
    delta = torch.randn(T, hid, generator=_gen(3)).to(dtype)
    w = 1 + 0.2 * torch.randn(hid, generator=_gen(4))
    want_h = h + delta.float()
    want = torch.from_numpy(P.rmsnorm(want_h.numpy(), w.numpy(), eps))
    hd, out = h.to(DEV), torch.empty(T, hid, dtype=dtype, device=DEV)
    ops().add_rmsnorm(hd, delta.to(DEV), w.to(DEV), eps, out)
    assert torch.allclose(hd.cpu(), want_h, atol=1e-6)
    assert (out.float().cpu() - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    # no delta, selected rows: h untouched
    rows = torch.tensor([18, 0, 7], dtype=torch.int32)
    hd2, out2 = h.to(DEV), torch.empty(3, hid, dtype=dtype, device=DEV)
    ops().add_rmsnorm(hd2, None, w.to(DEV), eps, out2, rows.to(DEV))
    want2 = torch.from_numpy(P.rmsnorm(h[rows.long()].numpy(), w.numpy(), eps))
    assert torch.equal(hd2.cpu(), h)
    assert (out2.float().cpu() - want2).abs().max() <= tol * max(1.0, float(want2.abs().max()))
    # delta and selected rows together
    out3 = torch.empty(3, hid, dtype=dtype, device=DEV)
    ops().add_rmsnorm(hd2, delta.to(DEV), w.to(DEV), eps, out3, rows.to(DEV))
    assert (out3.float().cpu() - want[rows.long()]).abs().max() <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("I", [100, 200])          # 200: the bfloat16 kernel with eight values per load
def test_swiglu_residual_convert(dtype, tol, I):
    T = 23
    gu = (torch.randn(T, 2 * I, generator=_gen(5)) * 2).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops().swiglu(gu.to(DEV), out)
    want = torch.from_numpy(P.swiglu(gu[:, :I].float().numpy(), gu[:, I:].float().numpy()))
    assert (out.float().cpu() - want).abs().max() <= tol * float(want.abs().max())
    h = torch.randn(T, I, generator=_gen(6))
    hd = h.to(DEV)
    ops().residual_add(hd, out)
    assert torch.allclose(hd.cpu(), h + out.float().cpu(), atol=1e-6)
    if dtype == torch.bfloat16:
        x = torch.randn(1000, generator=_gen(7))
        y = torch.empty(1000, dtype=torch.bfloat16, device=DEV)
        ops().convert(x.to(DEV), y)
        assert torch.equal(y.cpu(), x.to(torch.bfloat16))
        z = torch.empty(1000, dtype=torch.float32, device=DEV)
        ops().convert(y, z)
        assert torch.equal(z.cpu(), x.to(torch.bfloat16).float())


def _paged(K, V, lens, n_pages, seed):
    """Scatter dense per-sequence keys/values [len, Hkv, D] into shuffled pages; returns pages and block table."""
    Hkv, D = K[0].shape[1:]
    order = torch.randperm(n_pages, generator=_gen(seed)).tolist()
    width = max(-(-n // 64) for n in lens)
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    kp = torch.randn(n_pages, Hkv, 64, D, generator=_gen(seed + 1)) * 5      # stale content in unused rows
    vp = torch.randn(n_pages, Hkv, 64, D, generator=_gen(seed + 2)) * 5
    for s, n in enumerate(lens):
        for b in range(-(-n // 64)):
            pg = order.pop()
            table[s, b] = pg
            m = min(64, n - 64 * b)
            kp[pg, :, :m] = K[s][64 * b: 64 * b + m].transpose(0, 1)
            vp[pg, :, :m] = V[s][64 * b: 64 * b + m].transpose(0, 1)
    return kp, vp, table


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("H,Hkv,D,rot", [(5, 5, 48, 48), (6, 2, 16, 16), (7, 1, 80, 32), (4, 4, 128, 0)])
def test_rope_kv_write(dtype, tol, H, Hkv, D, rot, pairing):
    """pairing 0: half-split pairs (j, j + rot/2), the reference's; pairing 1: interleaved pairs (2j, 2j + 1)."""
    lens_before, new = [3, 70, 0], [5, 1, 66]
    B = 3
    T = sum(new)
    qkv = torch.randn(T, (H + 2 * Hkv) * D, generator=_gen(8)).to(dtype)
    positions = torch.cat([torch.arange(a, a + n) for a, n in zip(lens_before, new)]).int()
    seq = torch.cat([torch.full((n,), s) for s, n in enumerate(new)]).int()
    n_pages = 8
    table = torch.tensor([[5, -1], [2, 7], [0, 3]], dtype=torch.int32)
    inv_freq = torch.from_numpy((1.0 / np.power(np.float32(5000.0), np.arange(rot // 2, dtype=np.float32) * 2 / max(rot, 1))).astype(np.float32)) if rot else None
    kp = torch.zeros(n_pages, Hkv, 64, D, dtype=dtype)
    vp = torch.zeros_like(kp)
    want_qkv, want_k, want_v = qkv.clone(), kp.clone(), vp.clone()
    E.rope_kv_write(want_qkv, positions, seq, table, inv_freq, rot, want_k, want_v, H, Hkv, D, pairing=pairing)
    d_qkv, d_k, d_v = qkv.to(DEV), kp.to(DEV), vp.to(DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().rope_kv_write(d_qkv, positions.to(DEV), seq.to(DEV), table.to(DEV), None if inv_freq is None else inv_freq.to(DEV),
                        rot, d_k, d_v, H, Hkv, D, err, pairing)
    assert int(err.item()) == 0
    q_cols = H * D
    assert (d_qkv.float().cpu()[:, :q_cols] - want_qkv.float()[:, :q_cols]).abs().max() <= tol * 4
    assert torch.equal(d_qkv.cpu()[:, q_cols:], qkv[:, q_cols:])                 # k and v columns of the input stay
    assert (d_k.float().cpu() - want_k.float()).abs().max() <= tol * 4
    assert torch.equal(d_v.cpu(), want_v)
    # queries only (a run that reads another run's cache): no page is written
    d_k2 = torch.zeros_like(d_k)
    d_qkv2 = qkv.to(DEV)
    ops().rope_kv_write(d_qkv2, positions.to(DEV), seq.to(DEV), table.to(DEV), None if inv_freq is None else inv_freq.to(DEV),
                        rot, None, None, H, Hkv, D, err, pairing)
    assert torch.equal(d_qkv2.cpu()[:, :q_cols], d_qkv.cpu()[:, :q_cols]) and float(d_k2.abs().sum()) == 0
    # a missing page is reported, not written through
    bad = table.clone(); bad[2, 1] = -1
    ops().rope_kv_write(qkv.to(DEV), positions.to(DEV), seq.to(DEV), bad.to(DEV), None if inv_freq is None else inv_freq.to(DEV),
                        rot, d_k, d_v, H, Hkv, D, err)
    assert int(err.item()) == 2


def _attention_case(H, Hkv, D, lens_before, new, window, seed, spike=True):
    """Dense q/k/v per sequence, the plain result for the NEW tokens, and everything paged for the kernels.
    With `spike`, one far key per sequence is made to dominate the last query of head 0, so that a kernel
    which loses that key (a wrong page, a window off by one, a split that is skipped) is far off."""
    rng = np.random.default_rng(seed)
    K, V, Q, want = [], [], [], []
    for a, n in zip(lens_before, new):
        L = a + n
        k = rng.standard_normal((L, Hkv, D)).astype(np.float32)
        v = rng.standard_normal((L, Hkv, D)).astype(np.float32)
        q = rng.standard_normal((L, H, D)).astype(np.float32)
        if spike and L > 3:
            far = (L - window if window and L > window else 1)          # the oldest key the last query may see
            far = max(far, 0)
            k[far, 0, :] = 0; k[far, 0, 0] = 8.0 * math.sqrt(D)
            q[L - 1, 0, :] = 0; q[L - 1, 0, 0] = 8.0 * math.sqrt(D)
        K.append(k); V.append(v); Q.append(q)
    return Q, K, V


def _run_attention(kind, dtype, H, Hkv, D, lens_before, new, window, seed=0, groups=1):
    o = ops()
    Q, K, V = _attention_case(H, Hkv, D, lens_before, new, window, seed)
    scale = 1.0 / math.sqrt(D)
    tdt = dtype
    Kt = [torch.from_numpy(k).to(tdt) for k in K]
    Vt = [torch.from_numpy(v).to(tdt) for v in V]
    Qt = [torch.from_numpy(q).to(tdt) for q in Q]
    want = []
    for q, k, v, a, n in zip(Qt, Kt, Vt, lens_before, new):
        full = P.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), scale, window=window)
        want.append(full[a: a + n].reshape(n, H * D))
    want = np.concatenate(want)
    lens = [a + n for a, n in zip(lens_before, new)]
    n_pages = sum(-(-n // 64) for n in lens) + 3
    kp, vp, table = _paged(Kt, Vt, lens, n_pages, seed + 10)
    kp, vp = kp.to(tdt), vp.to(tdt)
    T = sum(new)
    # q as a view into a wider qkv-like buffer (row stride > H*D), as the engine passes it
    stride = (H + 2 * Hkv) * D
    qkv = torch.zeros(T, stride, dtype=tdt)
    qkv[:, : H * D] = torch.cat([q[a: a + n].reshape(n, H * D) for q, a, n in zip(Qt, lens_before, new)])
    positions = torch.cat([torch.arange(a, a + n) for a, n in zip(lens_before, new)]).int()
    seq = torch.cat([torch.full((n,), s) for s, n in enumerate(new)]).int()
    cu = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32)
    out = torch.full((T, H * D), float("nan"), dtype=tdt, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    d = lambda t: t.to(DEV)
    if kind == "generic":
        o.attention_generic(d(qkv), stride, d(kp), d(vp), d(table), d(positions), d(seq), out, H, Hkv, D, scale, window, err)
    elif kind == "prefill":
        n_tiles = sum(-(-n // 64) for n in new)
        o.attention_prefill_bf16(d(qkv), stride, d(kp), d(vp), d(table), d(positions), d(cu), n_tiles, out, H, Hkv, D, scale,
                                 window, err)
    elif kind == "prefill_tc":
        n_tiles = sum(-(-n // 128) for n in new)
        o.attention_prefill_tc_bf16(d(qkv), stride, d(kp), d(vp), d(table), d(positions), d(cu), n_tiles, out, H, Hkv, D, scale,
                                    window, err, groups)
    elif kind == "prefill_ws":
        o.attention_prefill_ws_bf16(d(qkv), stride, d(kp), d(vp), d(table), d(positions), d(cu), cu.tolist(), out, H, Hkv, D, scale,
                                    window, err, groups)
    else:
        B = len(new)
        n_splits = o.decode_splits(B, Hkv, H // Hkv, table.shape[1])
        for splits in sorted({1, n_splits, min(3, table.shape[1])}):
            partial = torch.full((B * H * splits * (D + 2),), float("nan"), device=DEV)
            counters = torch.zeros(B * H, dtype=torch.int32, device=DEV)
            out.fill_(float("nan"))
            o.attention_decode_bf16(d(qkv), stride, d(kp), d(vp), d(table), d(positions), out, partial, counters, H, Hkv, D,
                                    splits, scale, window, err)
            assert int(counters.abs().sum().item()) == 0            # the counters are left ready for the next launch
            got = out.float().cpu().numpy()
            assert np.abs(got - want).max() <= 2e-2, (splits, float(np.abs(got - want).max()))
    assert int(err.item()) == 0
    return out.float().cpu().numpy(), want


SHAPES = [(4, 2, 16), (3, 1, 32), (5, 5, 48), (9, 3, 64), (6, 2, 80), (7, 7, 96), (10, 1, 112), (8, 2, 128)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,Hkv,D", SHAPES + [(2, 1, 144), (2, 2, 256)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_generic(dtype, tol, H, Hkv, D, window):
    got, want = _run_attention("generic", dtype, H, Hkv, D, [0, 130, 63, 0, 200], [100, 3, 2, 1, 1], window)
    assert np.isfinite(got).all() and np.abs(got - want).max() <= tol


@pytest.mark.parametrize("H,Hkv,D", SHAPES)
@pytest.mark.parametrize("window", [0, 70, 64])
def test_attention_prefill_bf16(H, Hkv, D, window):
    # whole prompts of awkward lengths, a continued sequence (chunked prefill), single tokens
    got, want = _run_attention("prefill", torch.bfloat16, H, Hkv, D, [0, 130, 63, 0, 200, 0], [200, 67, 2, 1, 1, 64], window)
    assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2


@pytest.mark.parametrize("H,Hkv", [(9, 3), (4, 4), (5, 1)])
@pytest.mark.parametrize("window", [0, 70, 64, 200])
@pytest.mark.parametrize("groups", [1, 2, 3, 4])
def test_attention_prefill_tcgen05(H, Hkv, window, groups):
    """The tensor-memory kernel (head size 64): prompts of awkward lengths around its 128-token tiles and 64-key
    blocks, a continued sequence, single tokens, one long prompt."""
    got, want = _run_attention("prefill_tc", torch.bfloat16, H, Hkv, 64, [0, 130, 63, 0, 200, 0, 0, 17],
                               [200, 67, 2, 1, 1, 128, 129, 600], window, groups=groups)
    assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2


# (heads, kv heads): three heads of a group per CTA; four; one head and three row tiles per CTA; two heads and two row tiles
@pytest.mark.parametrize("H,Hkv", [(9, 3), (4, 1), (5, 5), (4, 2), (5, 1)])
@pytest.mark.parametrize("window", [0, 70, 64, 200])
@pytest.mark.parametrize("cluster", [0, 1, 2, 3, 5, 8])
def test_attention_prefill_warp_specialised(H, Hkv, window, cluster):
    """The warp-specialised tensor-memory kernel (head size 64): prompts of awkward lengths around its 128-token tiles and
    64-key blocks, a continued sequence, single tokens, long prompts whose tile groups are walked in pairs, and every way of
    dealing the key blocks out to a cluster."""
    got, want = _run_attention("prefill_ws", torch.bfloat16, H, Hkv, 64, [0, 130, 63, 0, 200, 0, 0, 17, 0],
                               [200, 67, 2, 1, 1, 128, 129, 600, 1100], window, groups=cluster)
    assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2


def test_attention_prefill_warp_specialised_with_more_sequences_than_its_launch_parameters_hold():
    """Twenty sequences in one step: the kernel then walks the offsets in device memory instead of its launch parameters."""
    news = [130, 1, 64, 200, 3, 128, 129, 65, 2, 300, 17, 90, 1, 256, 63, 127, 5, 400, 31, 77]
    before = [0, 700, 0, 130, 63, 0, 0, 17, 200, 0, 0, 64, 1000, 0, 1, 0, 321, 0, 0, 50]
    for cluster in (0, 1, 4):
        got, want = _run_attention("prefill_ws", torch.bfloat16, 6, 2, 64, before, news, 0, groups=cluster, seed=3)
        assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_attention_prefill_warp_specialised_at_random_shapes(seed):
    """Forty random steps per seed (heads and groups, one to five sequences of new and cached tokens of any length, windows,
    table widths beyond the need, every cluster size) against the generic kernel in float32 on the same bfloat16 inputs; the
    generic kernel is itself compared with the plain implementation in test_attention_generic."""
    o = ops()
    rng = np.random.default_rng(seed)
    for case in range(40):
        Hkv = int(rng.integers(1, 5)); G = int(rng.choice([1, 2, 3, 4, 6])); H = Hkv * G; D = 64
        B = int(rng.integers(1, 6))
        news = [int(rng.integers(1, 900)) for _ in range(B)]
        if rng.random() < 0.3:
            news[0] = int(rng.integers(900, 2600))
        before = [int(rng.integers(0, 1500)) if rng.random() < 0.4 else 0 for _ in range(B)]
        window = int(rng.choice([0, 0, 0, 64, 70, 300, 1000]))
        cluster = int(rng.choice([0, 0, 1, 2, 3, 4, 5, 6, 7, 8]))
        lens = [a + n for a, n in zip(before, news)]
        n_pages = sum(-(-L // 64) for L in lens) + 2
        width = max(-(-L // 64) for L in lens) + int(rng.integers(0, 3))
        perm = rng.permutation(n_pages)
        table = np.full((B, width), -1, dtype=np.int32)
        k = 0
        for s_, L in enumerate(lens):
            for b in range(-(-L // 64)):
                table[s_, b] = perm[k]; k += 1
        g = _gen(1000 * seed + case)
        kp = torch.randn(n_pages, Hkv, 64, D, generator=g).to(torch.bfloat16).to(DEV)
        vp = torch.randn(n_pages, Hkv, 64, D, generator=g).to(torch.bfloat16).to(DEV)
        T = sum(news)
        stride = (H + 2 * Hkv) * D
        qkv = (torch.randn(T, stride, generator=g) * (1.0 + 2.0 * rng.random())).to(torch.bfloat16).to(DEV)
        positions = torch.cat([torch.arange(a, a + n) for a, n in zip(before, news)]).int().to(DEV)
        seq = torch.cat([torch.full((n,), s_) for s_, n in enumerate(news)]).int().to(DEV)
        cu = torch.tensor([0] + list(np.cumsum(news)), dtype=torch.int32)
        tb = torch.from_numpy(table).to(DEV)
        scale = 1.0 / math.sqrt(D)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        o.attention_prefill_ws_bf16(qkv, stride, kp, vp, tb, positions, cu.to(DEV), cu.tolist(), out, H, Hkv, D, scale, window, err, cluster)
        ref = torch.full((T, H * D), float("nan"), dtype=torch.float32, device=DEV)
        o.attention_generic(qkv.float(), stride, kp.float(), vp.float(), tb, positions, seq, ref, H, Hkv, D, scale, window, err)
        what = (case, H, Hkv, news, before, window, cluster)
        assert int(err.item()) == 0, what
        assert torch.isfinite(out.float()).all(), what
        assert float((out.float() - ref).abs().max()) <= 3e-2, what


def test_attention_prefill_warp_specialised_moves_its_reference_maximum():
    """Scores that grow along the keys by far more than the gap the kernel lets its reference maximum lag behind: the rows'
    sums in tensor memory are rescaled several times."""
    o = ops()
    H = Hkv = 1
    D, L = 64, 700
    rng = np.random.default_rng(5)
    k = rng.standard_normal((L, Hkv, D)).astype(np.float32)
    v = rng.standard_normal((L, Hkv, D)).astype(np.float32)
    q = rng.standard_normal((L, H, D)).astype(np.float32)
    k[:, 0, 0] = np.arange(L) * 0.35                       # with q[.., 0] = 8: the raw score grows by 2.8 per key, 180 per block
    q[:, 0, 0] = 8.0
    scale = 1.0 / math.sqrt(D)
    bf = torch.bfloat16
    Kt, Vt, Qt = [torch.from_numpy(k).to(bf)], [torch.from_numpy(v).to(bf)], torch.from_numpy(q).to(bf)
    want = P.attention(Qt.float().numpy(), Kt[0].float().numpy(), Vt[0].float().numpy(), scale).reshape(L, H * D)
    kp, vp, table = _paged(Kt, Vt, [L], 14, 3)
    out = torch.full((L, H * D), float("nan"), dtype=bf, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, L], dtype=torch.int32)
    for cluster in (1, 2):
        o.attention_prefill_ws_bf16(Qt.reshape(L, H * D).to(DEV), H * D, kp.to(bf).to(DEV), vp.to(bf).to(DEV), table.to(DEV),
                                    torch.arange(L, dtype=torch.int32, device=DEV), cu.to(DEV), [0, L], out, H, Hkv, D, scale, 0, err, cluster)
        assert int(err.item()) == 0
        got = out.float().cpu().numpy()
        assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-2


@pytest.mark.parametrize("H,Hkv,D", SHAPES + [(12, 1, 64), (16, 16, 64)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_decode_bf16(H, Hkv, D, window):
    _run_attention("decode", torch.bfloat16, H, Hkv, D, [0, 63, 64, 130, 700, 1], [1, 1, 1, 1, 1, 1], window)


def test_attention_reports_a_missing_page():
    o = ops()
    H, Hkv, D = 2, 1, 16
    kp = torch.zeros(4, Hkv, 64, D, device=DEV)
    table = torch.tensor([[1, -1]], dtype=torch.int32, device=DEV)
    q = torch.zeros(1, H * D, device=DEV)
    out = torch.empty(1, H * D, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.attention_generic(q, H * D, kp, kp, table, torch.tensor([70], dtype=torch.int32, device=DEV),
                        torch.tensor([0], dtype=torch.int32, device=DEV), out, H, Hkv, D, 1.0, 0, err)
    assert int(err.item()) == 3


# (vocabulary, rows): one CTA per row with the row's probabilities in shared memory; a cluster of eight CTAs per row
# (large vocabulary, few rows), once with a vocabulary that is no multiple of its slices; one CTA per row without the
# shared-memory copy (many rows of a vocabulary too large for it)
@pytest.mark.parametrize("V,R", [(1000, 6), (49152 + 7, 6), (60011, 6), (60011, 70)])
def test_sampling(V, R):
    o = ops()
    rng = np.random.default_rng(V)
    logits = (rng.standard_normal((R, V)) * 2).astype(np.float32)
    logits[0, 17] = logits[0, 400] = logits[0].max() + 1          # a tie: the lower index wins
    logits[1, :5] = np.nan
    logits[2, :] = np.nan                                         # nothing to choose from
    logits[3, 10] = np.inf
    temperature = np.concatenate([[0.0, 0.0, 0.0, 0.0, 0.8, 1.3], rng.uniform(0.5, 1.5, R - 6)]).astype(np.float32)
    top_p = np.concatenate([[0.9, 0.9, 0.9, 0.9, 1.0, 0.6], rng.uniform(0.3, 1.0, R - 6)]).astype(np.float32)
    seed = np.concatenate([[1, 2, 3, 4, 1234, 99], rng.integers(0, 1000, R - 6)]).astype(np.int64)
    stream = np.arange(R, dtype=np.int64)
    dl = torch.from_numpy(logits).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    mism = 0
    for step in range(40 if R == 6 else 3):
        steps = np.full(R, step, dtype=np.int64)
        o.sample(dl, torch.from_numpy(temperature).to(DEV), torch.from_numpy(top_p).to(DEV), torch.from_numpy(seed).to(DEV),
                 torch.from_numpy(stream).to(DEV), torch.from_numpy(steps).to(DEV), out)
        got = out.cpu().numpy()
        assert got[0] == 17 and got[1] == int(np.nanargmax(logits[1])) and got[2] == -1 and got[3] == 10
        for r in range(4, R):
            want = P.sample_top_p(logits[r], float(temperature[r]), float(top_p[r]), P.uniform01(int(seed[r]), int(stream[r]), step))
            mism += int(got[r] != want)
    assert mism == 0
    # a strided view of a wider buffer works too
    wide = torch.zeros(R, V + 9, device=DEV)
    wide[:, :V] = dl
    o.sample(wide[:, :V], None, None, None, None, None, out)
    assert out.cpu().numpy()[0] == 17


@pytest.mark.parametrize("V", [49152, 16000 + 3])
def test_sampling_rows_that_stress_the_nucleus_search(V):
    """Rows made for the cluster sampler's search: all logits equal (every token ties with the nucleus' last member, nothing is
    ever left out of the candidates), two plateaus whose boundary is the threshold, a row so flat that thousands of
    probabilities stay between the bounds (more than the candidate list holds, so the exchanges go on), a row with one
    dominant token, a row with a few -inf and NaN logits, a threshold far below the largest probability.  Token for token
    against the plain sampler."""
    o = ops()
    rng = np.random.default_rng(V)
    rows = []
    rows.append((np.zeros(V, dtype=np.float32), 1.0, 0.5))
    two = np.zeros(V, dtype=np.float32); two[: V // 3] = 1.0
    rows.append((two, 0.9, 0.35))
    rows.append((two.copy(), 0.9, 0.8))
    rows.append(((rng.standard_normal(V) * 0.01).astype(np.float32), 1.0, 0.9))
    rows.append(((rng.standard_normal(V) * 0.01).astype(np.float32), 1.0, 0.999))
    peak = (rng.standard_normal(V)).astype(np.float32); peak[123] = 30.0
    rows.append((peak, 0.7, 0.9))
    holes = (rng.standard_normal(V) * 3).astype(np.float32); holes[5:50] = -np.inf; holes[60:70] = np.nan
    rows.append((holes, 1.2, 0.97))
    rows.append(((rng.standard_normal(V) * 6).astype(np.float32), 2.5, 0.9999))
    R = len(rows)
    logits = np.stack([r[0] for r in rows])
    temperature = np.array([r[1] for r in rows], dtype=np.float32)
    top_p = np.array([r[2] for r in rows], dtype=np.float32)
    seed = np.arange(100, 100 + R, dtype=np.int64)
    stream = np.arange(R, dtype=np.int64)
    dl = torch.from_numpy(logits).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    for step in range(12):
        steps = np.full(R, step, dtype=np.int64)
        o.sample(dl, torch.from_numpy(temperature).to(DEV), torch.from_numpy(top_p).to(DEV), torch.from_numpy(seed).to(DEV),
                 torch.from_numpy(stream).to(DEV), torch.from_numpy(steps).to(DEV), out)
        got = out.cpu().numpy()
        for r in range(R):
            want = P.sample_top_p(logits[r], float(temperature[r]), float(top_p[r]), P.uniform01(int(seed[r]), int(stream[r]), step))
            assert got[r] == want, (r, step, int(got[r]), int(want))


def test_sampled_distribution():
    o = ops()
    probs = np.array([0.5, 0.25, 0.125, 0.0625, 0.0625], dtype=np.float32)
    R = 4096
    logits = torch.from_numpy(np.log(probs)).repeat(R, 1).to(DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ones = torch.ones(R, device=DEV)
    o.sample(logits, ones, ones, torch.full((R,), 7, dtype=torch.int64, device=DEV), torch.arange(R, dtype=torch.int64, device=DEV),
             torch.zeros(R, dtype=torch.int64, device=DEV), out)
    freq = np.bincount(out.cpu().numpy(), minlength=5) / R
    assert np.abs(freq - probs).max() < 0.03
    o.sample(logits, ones, ones * 0.7, torch.full((R,), 7, dtype=torch.int64, device=DEV), torch.arange(R, dtype=torch.int64, device=DEV),
             torch.zeros(R, dtype=torch.int64, device=DEV), out)
    freq = np.bincount(out.cpu().numpy(), minlength=5) / R
    assert freq[2:].sum() == 0 and abs(freq[0] - 2 / 3) < 0.03       # nucleus of 0.7 = the two most probable tokens


# ------------------------------------------------------------------------------------------ weight-streaming products
def _bf(t):
    return t.to(torch.bfloat16)


def _rms_ref(h, w, eps):
    return _bf(torch.from_numpy(P.rmsnorm(h.numpy(), w.numpy(), eps)))


@pytest.fixture(params=["register-fed", "ring-two-ctas", "ring-two-pipelines"])
def skinny_kernel(request):
    """Both weight-streaming kernels, forced: the one that fetches weights into registers (what small matrices take) and the
    one that streams them through a ring in shared memory (large matrices, at most 32 rows), the latter in both its forms for
    up to 16 rows: two CTAs per SM, or one CTA whose two pipelines share the staged rows."""
    o = ops()
    o.skinny_variant({"register-fed": 1, "ring-two-ctas": 4, "ring-two-pipelines": 3}[request.param])
    yield request.param
    o.skinny_variant(0)


def _ring_takes(kernel, M):
    if kernel.startswith("ring") and M > 32:
        pytest.skip("the ring kernel takes at most 32 rows")


@pytest.mark.parametrize("M", [1, 8, 17, 64])
@pytest.mark.parametrize("N,K", [(72, 64), (576, 576), (200, 160), (576, 1536), (4752, 96), (3000, 1056), (5200, 2080)])   # (the last three: CTAs take several column tiles)
def test_skinny_linear(M, N, K, skinny_kernel):
    _ring_takes(skinny_kernel, M)
    o = ops()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = _bf(torch.randn(M, K, generator=_gen(M + N)))
    w = _bf(torch.randn(N, K, generator=_gen(K)) * 0.1)
    want = x.float() @ w.float().t()
    tol = 2e-2 * float(want.abs().max())
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.skinny_linear(x.to(DEV), None, w.to(DEV), out, err=err)
    assert (out.float().cpu() - want).abs().max() <= tol
    out32 = torch.full((M, N + 3), float("nan"), device=DEV)                 # a strided float32 output (logits)
    o.skinny_linear(x.to(DEV), None, w.to(DEV), out32[:, :N], err=err)
    assert (out32[:, :N].cpu() - want).abs().max() <= 1e-3 * max(1.0, float(want.abs().max()))
    assert torch.isnan(out32[:, N:]).all()
    h = torch.randn(M, N, generator=_gen(5))
    hd = h.to(DEV)
    o.skinny_linear(x.to(DEV), None, w.to(DEV), None, residual=hd, err=err)
    assert (hd.cpu() - (h + want)).abs().max() <= 1e-3 * max(1.0, float(want.abs().max()))
    # the norm as prologue
    hres = torch.randn(M, K, generator=_gen(6)) * 2
    nw = 1 + 0.1 * torch.randn(K, generator=_gen(7))
    xn = _rms_ref(hres, nw, 1e-5)
    want_n = xn.float() @ w.float().t()
    o.skinny_linear(hres.to(DEV), (nw.to(DEV), 1e-5), w.to(DEV), out, err=err)
    assert (out.float().cpu() - want_n).abs().max() <= 2e-2 * float(want_n.abs().max())
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,N,K", [(8, 2304, 2048), (16, 640, 8192), (40, 2304, 2048), (2, 1200, 2048), (3, 1200, 2048)])
def test_skinny_linear_chooses_its_kernel_by_size(M, N, K):
    """Left to themselves the launchers take the ring kernel from 9 MB of weights and up to 32 rows (from 4.5 MB for one or two
    rows: the last two cases lie on either side); where it does not take the
    sizes (16 rows of K = 8,192 do not fit its shared memory beside two stages; 40 rows are too many) they fall back to the
    register-fed kernel.  Same result either way."""
    o = ops()
    o.skinny_variant(0)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    x = _bf(torch.randn(M, K, generator=_gen(M)))
    w = _bf(torch.randn(N, K, generator=_gen(N)) * 0.05)
    h = torch.randn(M, N, generator=_gen(K))
    want = h + x.float() @ w.float().t()
    hd = h.to(DEV)
    o.skinny_linear(x.to(DEV), None, w.to(DEV), None, residual=hd, err=err)
    assert (hd.cpu() - want).abs().max() <= 1e-3 * max(1.0, float(want.abs().max()))
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,I,K", [(3, 192, 64), (8, 1536, 576), (33, 160, 96), (64, 1000, 1536), (5, 5000, 96), (20, 2000, 1088), (16, 3000, 3104),
                                   (32, 2504, 1024)])
def test_skinny_swiglu(M, I, K, skinny_kernel):
    _ring_takes(skinny_kernel, M)
    o = ops()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    hres = torch.randn(M, K, generator=_gen(M)) * 2
    nw = 1 + 0.1 * torch.randn(K, generator=_gen(I))
    w = _bf(torch.randn(2 * I, K, generator=_gen(K)) * 0.2)
    xn = _rms_ref(hres, nw, 1e-6)
    gu = xn.float() @ w.float().t()
    want = torch.from_numpy(P.swiglu(gu[:, :I].numpy(), gu[:, I:].numpy()))
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.skinny_swiglu(hres.to(DEV), (nw.to(DEV), 1e-6), w.to(DEV), out, err=err)
    assert (out.float().cpu() - want).abs().max() <= 2e-2 * float(want.abs().max())
    o.skinny_swiglu(xn.to(DEV), None, w.to(DEV), out, err=err)
    assert (out.float().cpu() - want).abs().max() <= 2e-2 * float(want.abs().max())
    assert int(err.item()) == 0


@pytest.mark.parametrize("H,Hkv,D,K,rot", [(4, 2, 16, 64, 16), (3, 1, 32, 96, 32), (9, 3, 64, 576, 64), (5, 5, 48, 160, 0), (2, 1, 128, 256, 128),
                                           (40, 8, 64, 96, 64), (32, 32, 64, 2048, 64)])   # (the last two: CTAs take several column tiles)
def test_skinny_qkv_rope(H, Hkv, D, K, rot, skinny_kernel):
    o = ops()
    lens_before, new = [3, 70, 0], [5, 1, 20]
    T = sum(new)
    hres = torch.randn(T, K, generator=_gen(H)) * 2
    nw = 1 + 0.1 * torch.randn(K, generator=_gen(D))
    w = _bf(torch.randn((H + 2 * Hkv) * D, K, generator=_gen(K)) * 0.2)
    positions = torch.cat([torch.arange(a, a + n) for a, n in zip(lens_before, new)]).int()
    seq = torch.cat([torch.full((n,), s) for s, n in enumerate(new)]).int()
    table = torch.tensor([[5, -1], [2, 7], [0, 3]], dtype=torch.int32)
    inv_freq = torch.from_numpy((1.0 / np.power(np.float32(5000.0), np.arange(rot // 2, dtype=np.float32) * 2 / max(rot, 1))).astype(np.float32)) if rot else None
    xn = _rms_ref(hres, nw, 1e-5)
    qkv = (xn.float() @ w.float().t())                                     # float32 reference all the way
    kp = torch.zeros(8, Hkv, 64, D); vp = torch.zeros_like(kp)
    E.rope_kv_write(qkv, positions, seq, table, inv_freq, rot, kp, vp, H, Hkv, D)
    dq = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    dk = torch.zeros(8, Hkv, 64, D, dtype=torch.bfloat16, device=DEV); dv = torch.zeros_like(dk)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.skinny_qkv_rope(hres.to(DEV), (nw.to(DEV), 1e-5), w.to(DEV), dq, positions.to(DEV), seq.to(DEV), table.to(DEV),
                      None if inv_freq is None else inv_freq.to(DEV), rot, dk, dv, H, Hkv, D, err)
    assert int(err.item()) == 0
    scale = float(qkv.abs().max())
    assert (dq.float().cpu() - qkv[:, : H * D]).abs().max() <= 2e-2 * scale
    assert (dk.float().cpu() - kp).abs().max() <= 2e-2 * scale
    assert (dv.float().cpu() - vp).abs().max() <= 2e-2 * scale
    assert float(dk.float().abs().sum()) > 0


# ------------------------------------------------------------------------------------------ tensor-core (tcgen05 + TMA) products
def _err_word():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("M", [17, 128, 300, 2048])
@pytest.mark.parametrize("N,K", [(64, 64), (576, 576), (200, 160), (960, 576), (576, 1536), (1000, 72)])
def test_tc_linear(M, N, K):
    o = ops()
    x = _bf(torch.randn(M, K, generator=_gen(M + N)))
    w = _bf(torch.randn(N, K, generator=_gen(K)) * 0.1)
    want = x.float() @ w.float().t()
    big = max(1.0, float(want.abs().max()))
    err = _err_word()
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.tc_linear(x.to(DEV), w.to(DEV), out, err=err)
    assert (out.float().cpu() - want).abs().max() <= 1e-2 * big
    out32 = torch.full((M, N + 5), float("nan"), device=DEV)                   # a strided float32 output
    o.tc_linear(x.to(DEV), w.to(DEV), out32[:, :N], err=err)
    assert (out32[:, :N].cpu() - want).abs().max() <= 2e-5 * big and torch.isnan(out32[:, N:]).all()
    h = torch.randn(M, N, generator=_gen(5))
    hd = h.to(DEV)
    o.tc_linear(x.to(DEV), w.to(DEV), None, residual=hd, err=err)
    assert (hd.cpu() - (h + want)).abs().max() <= 2e-5 * big
    # x as a view with a row pitch (a slice of a wider buffer)
    wide = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x.to(DEV)
    o.tc_linear(wide[:, :K], w.to(DEV), out, err=err)
    assert (out.float().cpu() - want).abs().max() <= 1e-2 * big
    assert int(err.item()) == 0


@pytest.mark.parametrize("M,I,K", [(40, 192, 64), (2048, 1536, 576), (129, 64, 96), (500, 2560, 960)])
def test_tc_swiglu(M, I, K):
    o = ops()
    x = _bf(torch.randn(M, K, generator=_gen(M)))
    w = _bf(torch.randn(2 * I, K, generator=_gen(K)) * 0.2)
    gu = x.float() @ w.float().t()
    want = torch.from_numpy(P.swiglu(gu[:, :I].numpy(), gu[:, I:].numpy()))
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = _err_word()
    o.tc_swiglu(x.to(DEV), w.to(DEV), out, err)
    assert int(err.item()) == 0
    assert (out.float().cpu() - want).abs().max() <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("H,Hkv,D,K,rot", [(9, 3, 64, 576, 64), (2, 1, 128, 256, 128), (3, 3, 64, 96, 0)])
def test_tc_qkv_rope(H, Hkv, D, K, rot):
    o = ops()
    lens_before, new = [3, 70, 0], [150, 1, 120]
    T = sum(new)
    x = _bf(torch.randn(T, K, generator=_gen(H)))
    w = _bf(torch.randn((H + 2 * Hkv) * D, K, generator=_gen(K)) * 0.2)
    positions = torch.cat([torch.arange(a, a + n) for a, n in zip(lens_before, new)]).int()
    seq = torch.cat([torch.full((n,), s) for s, n in enumerate(new)]).int()
    table = torch.tensor([[5, 1, 9], [2, 7, -1], [0, 3, -1]], dtype=torch.int32)
    inv_freq = torch.from_numpy((1.0 / np.power(np.float32(5000.0), np.arange(rot // 2, dtype=np.float32) * 2 / max(rot, 1))).astype(np.float32)) if rot else None
    qkv = x.float() @ w.float().t()
    kp = torch.zeros(10, Hkv, 64, D); vp = torch.zeros_like(kp)
    E.rope_kv_write(qkv, positions, seq, table, inv_freq, rot, kp, vp, H, Hkv, D)
    dq = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    dk = torch.zeros(10, Hkv, 64, D, dtype=torch.bfloat16, device=DEV); dv = torch.zeros_like(dk)
    err = _err_word()
    o.tc_qkv_rope(x.to(DEV), w.to(DEV), dq, positions.to(DEV), seq.to(DEV), table.to(DEV),
                  None if inv_freq is None else inv_freq.to(DEV), rot, dk, dv, H, Hkv, D, err)
    assert int(err.item()) == 0
    scale = float(qkv.abs().max())
    assert (dq.float().cpu() - qkv[:, : H * D]).abs().max() <= 1e-2 * scale
    assert (dk.float().cpu() - kp).abs().max() <= 1e-2 * scale
    assert (dv.float().cpu() - vp).abs().max() <= 1e-2 * scale
