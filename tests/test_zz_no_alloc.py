"""The decode attention entry point that allocates nothing (csrc/velomind_no_alloc.h), called through its
exported C symbol and compared with the ordinary entry point.

Some callers of this library cannot call cudaMalloc: a plugin inside a host program with a frozen memory
budget, or code at a point where an allocation would stall the device.  For them the library keeps the
kernel's scratch in a static device array.  This test makes two calls in a row and checks both, bit for bit, against the
ordinary entry point (whose scratch the test allocates itself): both entries run the same kernel, so this is a test of
the wiring (the symbol's address, the layout of the scratch, the clearing of the counters), not of the kernel's
arithmetic, which tests/test_kernels_gpu.py compares with a plain function.  Before each call the whole static array is
filled with garbage (all bits set: NaN partials, non-zero counters), so a call that relied on an earlier call's leftovers,
or that did not clear its counters, would fail.  The file sorts last on purpose: if it fails, a run that stops at the first
failure has already run every other test.  It passes alone in a fresh process and after the other tests.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(B, H, Hkv, D, lens, seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    n_pages = sum(-(-n // 64) for n in lens) + 2
    kp = torch.randn(n_pages, Hkv, 64, D, generator=g).to(torch.bfloat16)
    vp = torch.randn(n_pages, Hkv, 64, D, generator=g).to(torch.bfloat16)
    width = max(-(-n // 64) for n in lens)
    table = torch.full((B, width), -1, dtype=torch.int32)
    order = torch.randperm(n_pages, generator=g).tolist()
    for s, n in enumerate(lens):
        for b in range(-(-n // 64)):
            table[s, b] = order.pop()
    q = torch.randn(B, H * D, generator=g).to(torch.bfloat16)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kp, vp, table, positions)]


def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row():
    from velomind_b200.kernels import ops
    from velomind_b200.kernels.library import library
    lib = library()
    fn = lib.vm_attention_decode_bf16_no_alloc
    fn.restype = ctypes.c_int
    need = lib.vm_attention_decode_no_alloc_bytes
    need.restype = ctypes.c_longlong
    c_int, c_f, c_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
    stream = c_p(torch.cuda.current_stream().cuda_stream)
    lib.vm_attention_decode_no_alloc_scratch.restype = c_p
    address = lib.vm_attention_decode_no_alloc_scratch()
    assert address

    class _Scratch:
        __cuda_array_interface__ = {"data": (int(address), False), "shape": (8 * 1024 * 1024,), "typestr": "|u1", "version": 2}

    scratch = torch.as_tensor(_Scratch(), device=DEV)

    for call, (B, H, Hkv, D, lens, splits) in enumerate([(5, 9, 3, 64, [1, 64, 130, 700, 65], 7),
                                                          (3, 8, 2, 128, [300, 2, 129], 3)]):
        q, kp, vp, table, positions = _case(B, H, Hkv, D, lens, seed=call)
        scale = 1.0 / math.sqrt(D)
        want = torch.empty(B, H * D, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(B * H * splits * (D + 2), device=DEV)
        counters = torch.zeros(B * H, dtype=torch.int32, device=DEV)
        ops.attention_decode_bf16(q, H * D, kp, vp, table, positions, want, partial, counters, H, Hkv, D, splits, scale)
        got = torch.full_like(want, float("nan"))
        assert need(B, H, D, splits) <= 8 * 1024 * 1024
        scratch.fill_(0xFF)                                  # garbage where the counters and the partials will lie
        torch.cuda.synchronize()
        rc = fn(c_p(q.data_ptr()), c_int(H * D), c_p(kp.data_ptr()), c_p(vp.data_ptr()), c_p(table.data_ptr()),
                c_int(table.shape[1]), c_p(positions.data_ptr()), c_p(got.data_ptr()), c_int(B), c_int(H), c_int(Hkv),
                c_int(D), c_int(splits), c_f(scale), c_int(0), c_int(kp.shape[0]), c_p(0), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)                        # the same kernel on the same inputs: the same bits

    # sizes the kernel does not take are refused before anything is put on the stream
    rc = fn(c_p(0), c_int(H * D), c_p(0), c_p(0), c_p(0), c_int(1), c_p(0), c_p(0), c_int(1), c_int(8), c_int(2), c_int(64), c_int(17),
            c_f(1.0), c_int(0), c_int(1), c_p(0), stream)
    assert rc == -1
    # a request beyond the static array is refused, and nothing runs
    B, H, D, splits = 64, 64, 128, 16
    assert need(B, H, D, splits) > 8 * 1024 * 1024
    rc = fn(c_p(0), c_int(H * D), c_p(0), c_p(0), c_p(0), c_int(1), c_p(0), c_p(0), c_int(B), c_int(H), c_int(H),
            c_int(D), c_int(splits), c_f(1.0), c_int(0), c_int(1), c_p(0), stream)
    assert rc == -3
