"""The kernel launchers of the library (include/velomind_b200/kernels.h) bound for Python: thin checked wrappers that take
torch CUDA tensors and launch on torch's current stream.  The kernel tests and the microbenchmark call the kernels alone
through these; the engine itself is C++ and calls the launchers directly (engine/ops.h).

There is no other implementation: a tensor that is not on a CUDA device, or a missing library, raises.  Activations are
float32 or bfloat16; the residual stream is always float32.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .library import KernelLibraryError, library

F32, BF16 = 0, 1
PAIR_HALF_SPLIT, PAIR_INTERLEAVED = 0, 1      # which two values of a head a rotary encoding turns together (csrc/common.cuh)
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

launch_count = 0          # this library's own kernels launched through this module (the bench reports it)
library_calls = 0         # library matrix products (cuBLAS through torch.mm)
h2d_bytes = 0             # bytes of step inputs copied from pinned host memory (descriptors, sampler parameters)
d2h_bytes = 0             # bytes of step results that reached the host (sampled tokens)
tc_attention_calls = 0    # launches of the tcgen05 prefill attention (tests check that long prompts take it)


# Debugging switches, read once from the environment (the reference has VELOMIND_CUDA_SYNC and VELOMIND_FAIL_BACKEND for
# the same purposes: src/cuda/cuda_context.cu:115-118, src/cuda/ops/backend_error.h:31-51).  Both act on the host only.
SYNC_EVERY_OP = os.environ.get("VELOMIND_B200_SYNC", "") == "1"    # wait for the device after every launch: an error names its op
FAIL_OP = os.environ.get("VELOMIND_B200_FAIL_OP", "")              # the op of this name raises after its launch (fault injection)


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} has no kernel (float32 and bfloat16 do)") from None


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return _c_p(0)
    if not t.is_cuda:
        raise KernelError("this library runs on CUDA devices only; got a tensor on " + str(t.device))
    return _c_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream's handle (the raw query is several times cheaper than building a Stream object)."""
    if _raw_stream is not None:
        return _c_p(_raw_stream(torch.cuda.current_device()))
    return _c_p(torch.cuda.current_stream().cuda_stream)


def _check(status: int, name: str) -> None:
    global launch_count
    launch_count += 1
    if status == 0:
        if FAIL_OP and name == FAIL_OP:
            raise KernelError(f"{name}: injected failure (VELOMIND_B200_FAIL_OP)")
        if SYNC_EVERY_OP:
            try:
                torch.cuda.synchronize()
            except RuntimeError as ex:
                raise KernelError(f"{name}: {ex}") from None
        return
    if status == -1:
        raise KernelError(f"{name}: this size or dtype is not supported by the kernel")
    if status == -2:
        raise KernelError(f"{name}: bad argument")
    raise KernelError(f"{name}: CUDA error {status}")


def _contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


# ------------------------------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = table[tokens[t], :] as float32.  table [V, hid] float32|bfloat16, tokens int32 [T]."""
    T, hid = out.shape
    _check(library().vm_embed_gather(_ptr(_contig(table, "table")), _c_int(dtype_code(table)), _ptr(tokens), _ptr(out),
                                     _c_int(T), _c_int(hid), _c_int(table.shape[0]), _ptr(err), _stream()), "embed_gather")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
    """h += delta (if given), out = rmsnorm(h) * weight.  h float32 [T, hid]; delta/out of the activation dtype;
    weight float32 [hid].  With `rows` (int32 [R]) only those rows are normed into out [R, hid] and h is not written."""
    n_out, hid = out.shape
    if weight.dtype != torch.float32 or h.dtype != torch.float32:
        raise KernelError("add_rmsnorm: residual and norm weight are float32")
    if delta is not None and delta.dtype != out.dtype:
        raise KernelError("add_rmsnorm: delta and out must share the activation dtype")
    _check(library().vm_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), _ptr(out), _ptr(rows), _c_int(n_out), _c_int(hid),
                                    _c_f(eps), _c_int(dtype_code(out)), _stream()), "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    """h += delta; h float32, delta of the activation dtype, same shape."""
    _check(library().vm_residual_add(_ptr(h), _ptr(_contig(delta, "delta")), _c_ll(h.numel()), _c_int(dtype_code(delta)),
                                     _stream()), "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]; gate_up [T, 2I], out [T, I]."""
    T, I = out.shape
    _check(library().vm_swiglu(_ptr(_contig(gate_up, "gate_up")), _ptr(out), _c_int(T), _c_int(I), _c_int(dtype_code(out)),
                               _stream()), "swiglu")


def convert(src: torch.Tensor, out: torch.Tensor) -> None:
    """out = src in out's dtype (float32 <-> bfloat16)."""
    _check(library().vm_convert(_ptr(_contig(src, "src")), _c_int(dtype_code(src)), _ptr(out), _c_int(dtype_code(out)),
                                _c_ll(src.numel()), _stream()), "convert")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], rot_dim: int, k_pages: Optional[torch.Tensor],
                  v_pages: Optional[torch.Tensor], H: int, Hkv: int, D: int, err: Optional[torch.Tensor] = None,
                  pairing: int = 0) -> None:
    """Rotate queries (in place) and keys of qkv [T, (H+2Hkv)*D]; write keys and values into the pages
    k_pages/v_pages [n_pages, Hkv, 64, D] at block_table[seq, pos // 64] (int32 [B, max_blocks]).
    With k_pages None only the queries are rotated (a run that reads another run's cache).
    pairing: PAIR_HALF_SPLIT (j, j + rot_dim/2) or PAIR_INTERLEAVED (2j, 2j + 1)."""
    T = qkv.shape[0]
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    _check(library().vm_rope_kv_write(_ptr(_contig(qkv, "qkv")), _ptr(positions), _ptr(seq_of_token), _ptr(block_table),
                                      _c_int(block_table.shape[1]), _ptr(inv_freq), _c_int(rot_dim), _c_int(pairing), _ptr(k_pages),
                                      _ptr(v_pages), _c_int(T), _c_int(H), _c_int(Hkv), _c_int(D),
                                      _c_int(n_pages), _c_int(dtype_code(qkv)), _ptr(err), _stream()), "rope_kv_write")


def attention_generic(q: torch.Tensor, q_row_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor, out: torch.Tensor,
                      H: int, Hkv: int, D: int, scale: float, window: int = 0, err: Optional[torch.Tensor] = None) -> None:
    """out[t, h*D:(h+1)*D] = attention of query (t, h) over its sequence's cached keys at positions
    max(0, pos-window+1)..pos (window 0: all).  q may be a view into qkv with row stride q_row_stride."""
    T = out.shape[0]
    _check(library().vm_attention_generic(_ptr(q), _c_int(q_row_stride), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                          _c_int(block_table.shape[1]), _ptr(positions), _ptr(seq_of_token), _ptr(out),
                                          _c_int(T), _c_int(H), _c_int(Hkv), _c_int(D), _c_f(scale), _c_int(window),
                                          _c_int(k_pages.shape[0]), _c_int(dtype_code(out)), _ptr(err), _stream()),
           "attention_generic")


def attention_prefill_bf16(q: torch.Tensor, q_row_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, positions: torch.Tensor, cu_tokens: torch.Tensor, n_tiles: int,
                           out: torch.Tensor, H: int, Hkv: int, D: int, scale: float, window: int = 0,
                           err: Optional[torch.Tensor] = None, groups: int = 1) -> None:
    """Tensor-core attention of the step's new tokens over the cache (bfloat16, D in 16..128 step 16).
    cu_tokens int32 [B+1]: token offsets of the sequences; n_tiles = sum of ceil(new tokens / 64);
    groups (1, 2, 4): warp groups sharing a tile's key blocks (for tiles that see many keys)."""
    B = cu_tokens.shape[0] - 1
    _check(library().vm_attention_prefill_bf16(_ptr(q), _c_int(q_row_stride), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                               _c_int(block_table.shape[1]), _ptr(positions), _ptr(cu_tokens), _c_int(B),
                                               _c_int(n_tiles), _ptr(out), _c_int(H), _c_int(Hkv), _c_int(D), _c_f(scale),
                                               _c_int(window), _c_int(k_pages.shape[0]), _ptr(err), _c_int(groups), _stream()),
           "attention_prefill_bf16")


def attention_prefill_tc_bf16(q: torch.Tensor, q_row_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                              block_table: torch.Tensor, positions: torch.Tensor, cu_tokens: torch.Tensor, n_tiles: int,
                              out: torch.Tensor, H: int, Hkv: int, D: int, scale: float, window: int = 0,
                              err: Optional[torch.Tensor] = None, groups: int = 1) -> None:
    """The same attention on tcgen05 (tensor-memory accumulators), head size 64 only: a CTA per 128 new tokens and
    head.  n_tiles = sum of ceil(new tokens / 128); groups (1, 2, 4): groups of 128 threads that take a tile's key
    blocks in turn."""
    global tc_attention_calls
    tc_attention_calls += 1
    B = cu_tokens.shape[0] - 1
    _check(library().vm_attention_prefill_tc_bf16(_ptr(q), _c_int(q_row_stride), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                                  _c_int(block_table.shape[1]), _ptr(positions), _ptr(cu_tokens), _c_int(B),
                                                  _c_int(n_tiles), _ptr(out), _c_int(H), _c_int(Hkv), _c_int(D), _c_f(scale),
                                                  _c_int(window), _c_int(k_pages.shape[0]), _ptr(err), _c_int(groups), _stream()),
           "attention_prefill_tc_bf16")


def attention_prefill_ws_bf16(q: torch.Tensor, q_row_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                              block_table: torch.Tensor, positions: torch.Tensor, cu_tokens: torch.Tensor, host_cu_tokens,
                              out: torch.Tensor, H: int, Hkv: int, D: int, scale: float, window: int = 0,
                              err: Optional[torch.Tensor] = None, groups: int = 0) -> None:
    """The warp-specialised tcgen05 attention (head size 64): a CTA per group of 128-row tiles that share a kv head,
    softmax warps, a copy warp (TMA) and a product warp; clusters of `groups` CTAs (0: chosen) take a pair of tile groups'
    key blocks in turn.  host_cu_tokens: the offsets of cu_tokens as a list of ints."""
    global tc_attention_calls
    tc_attention_calls += 1
    B = cu_tokens.shape[0] - 1
    host = (ctypes.c_int * (B + 1))(*[int(x) for x in host_cu_tokens])
    _check(library().vm_attention_prefill_ws_bf16(_ptr(q), _c_int(q_row_stride), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                                  _c_int(block_table.shape[1]), _ptr(positions), _ptr(cu_tokens), host, _c_int(B),
                                                  _ptr(out), _c_int(H), _c_int(Hkv), _c_int(D), _c_f(scale), _c_int(window),
                                                  _c_int(k_pages.shape[0]), _ptr(err), _c_int(groups), _stream()),
           "attention_prefill_ws_bf16")


_decode_counters = {}
DECODE_COUNTERS = 1 << 16
MAX_DECODE_SPLITS = 16


def decode_counters(device) -> torch.Tensor:
    """Zeroed int32 counters the split-KV decode kernel leaves zero after every launch (one per device)."""
    key = str(device)
    if key not in _decode_counters:
        _decode_counters[key] = torch.zeros(DECODE_COUNTERS, dtype=torch.int32, device=device)
    return _decode_counters[key]


DECODE_ONE_CTA_BLOCKS = 16     # block tables up to this wide (1,024 tokens): at most two rounds of pages for ten warps


def decode_splits(B: int, Hkv: int, G: int, table_width: int, device=None) -> int:
    """How many CTAs share the keys of one (sequence, kv head): enough to fill the GPU, a function of the
    step's SHAPE only (so that a captured launch stays valid as sequences grow)."""
    groups = B * Hkv * (-(-G // 16))          # a CTA serves up to 16 query heads of one kv head
    sms = sm_count(device)
    if groups <= sms and table_width <= DECODE_ONE_CTA_BLOCKS:
        return 1                              # short sequences: one CTA of ten warps holds all pages, nothing is merged across CTAs
    want = -(-sms // groups)                  # about one CTA per SM ...
    table_width = max(1, table_width // 4)    # ... and at least a page per warp of a CTA (the width bounds the pages)
    return max(1, min(want, MAX_DECODE_SPLITS, table_width))


def attention_decode_bf16(q: torch.Tensor, q_row_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                          block_table: torch.Tensor, positions: torch.Tensor, out: torch.Tensor, partial: torch.Tensor,
                          counters: torch.Tensor, H: int, Hkv: int, D: int, n_splits: int, scale: float, window: int = 0,
                          err: Optional[torch.Tensor] = None) -> None:
    """One new token per sequence: split-KV attention over the cache (bfloat16, D <= 128, D % 8 == 0).
    partial: float32 scratch of B*H*n_splits*(D+2); counters: zeroed int32, left zero."""
    B = out.shape[0]
    if partial.numel() < B * H * n_splits * (D + 2) or counters.numel() < B * H:
        raise KernelError("attention_decode_bf16: scratch too small")
    _check(library().vm_attention_decode_bf16(_ptr(q), _c_int(q_row_stride), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                                              _c_int(block_table.shape[1]), _ptr(positions), _ptr(out), _ptr(partial),
                                              _ptr(counters), _c_int(B), _c_int(H), _c_int(Hkv), _c_int(D), _c_int(n_splits),
                                              _c_f(scale), _c_int(window), _c_int(k_pages.shape[0]), _ptr(err), _stream()),
           "attention_decode_bf16")


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of `device` (the current one if None), asked once."""
    key = str(device) if device is not None else "current"
    if key not in _sm_counts:
        dev = device if device is not None else torch.cuda.current_device()
        _sm_counts[key] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_counts[key]


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out = x @ weight^T through torch (cuBLAS): the library product the microbenchmark compares this library's kernels with.
    x [T, K], weight [N, K], out [T, N]; float32 runs without any reduced-precision mode."""
    if not x.is_cuda:
        raise KernelError("this library runs on CUDA devices only; got a tensor on " + str(x.device))
    global library_calls
    library_calls += 1
    if x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise KernelError("float32 matrix products must not use TF32; torch.backends.cuda.matmul.allow_tf32 is set")
    if out.dtype == x.dtype:
        torch.mm(x, weight.t(), out=out)
    else:
        torch.mm(x, weight.t(), out_dtype=out.dtype, out=out)


def _norm_args(norm):
    if norm is None:
        return 0, None, 0.0
    weight, eps = norm
    return 1, weight, float(eps)


def skinny_variant(variant: int) -> None:
    """Which weight-streaming kernel the three launchers below take: 0 by size, 1 the register-fed one, 2 the one that streams
    the weights through shared memory (refuses what it does not take), 3 / 4 that one as one CTA with two pipelines / as two CTAs
    per SM."""
    library().vm_skinny_variant(_c_int(variant))


def skinny_linear(x: torch.Tensor, norm, weight: torch.Tensor, out: Optional[torch.Tensor],
                  residual: Optional[torch.Tensor] = None, err: Optional[torch.Tensor] = None) -> None:
    """out = x' W^T (bf16 or float32 out), or residual += x' W^T (float32), for M <= 64 rows.
    x' = x (bf16 [M, K]) when `norm` is None, else rmsnorm(x) * norm[0] with eps norm[1] from x float32 [M, K]."""
    M, K = x.shape
    N = weight.shape[0]
    pro, nw, eps = _norm_args(norm)
    _check(library().vm_skinny_linear(_ptr(_contig(x, "x")), _c_int(pro), _ptr(nw), _c_f(eps), _ptr(weight), _c_int(M), _c_int(N),
                                      _c_int(K), _ptr(out), _c_int(out.stride(0) if out is not None else N),
                                      _c_int(1 if (out is not None and out.dtype == torch.float32) else 0), _ptr(residual),
                                      _ptr(err), _stream()), "skinny_linear")


def skinny_swiglu(x: torch.Tensor, norm, weight: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out[M, I] = silu(x' Wg^T) * (x' Wu^T), weight = [Wg; Wu] stacked [2I, K]; x' as in skinny_linear."""
    M, K = x.shape
    pro, nw, eps = _norm_args(norm)
    _check(library().vm_skinny_swiglu(_ptr(_contig(x, "x")), _c_int(pro), _ptr(nw), _c_f(eps), _ptr(weight), _c_int(M),
                                      _c_int(out.shape[1]), _c_int(K), _ptr(_contig(out, "out")), _ptr(err), _stream()), "skinny_swiglu")


def skinny_qkv_rope(x: torch.Tensor, norm, weight: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                    seq_of_token: torch.Tensor, block_table: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dim: int,
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], H: int, Hkv: int, D: int,
                    err: Optional[torch.Tensor] = None, pairing: int = 0) -> None:
    """q_out[M, H*D] = rotated queries; rotated keys and values go straight into the cache pages.
    weight = [Wq; Wk; Wv] stacked; x' as in skinny_linear; rot_dim 0 or D; half-split pairing only."""
    M, K = x.shape
    pro, nw, eps = _norm_args(norm)
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    _check(library().vm_skinny_qkv_rope(_ptr(_contig(x, "x")), _c_int(pro), _ptr(nw), _c_f(eps), _ptr(weight), _c_int(M), _c_int(K),
                                        _ptr(_contig(q_out, "q_out")), _ptr(positions), _ptr(seq_of_token), _ptr(block_table),
                                        _c_int(block_table.shape[1]), _ptr(inv_freq), _c_int(rot_dim), _c_int(pairing), _ptr(k_pages),
                                        _ptr(v_pages), _c_int(H), _c_int(Hkv), _c_int(D), _c_int(n_pages), _ptr(err), _stream()),
           "skinny_qkv_rope")


def tc_linear(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor], residual: Optional[torch.Tensor] = None,
              err: Optional[torch.Tensor] = None) -> None:
    """out = x W^T (bf16 or float32 out) or residual += x W^T (float32), on tcgen05 tensor cores.
    x bf16 [M, K] with unit column stride (rows may be strided), weight bf16 [N, K]."""
    M, K = x.shape
    N = weight.shape[0]
    if x.stride(1) != 1:
        raise KernelError("tc_linear: x must have unit column stride")
    _check(library().vm_tc_linear(_ptr(x), _c_ll(x.stride(0)), _ptr(weight), _c_int(M), _c_int(N), _c_int(K), _ptr(out),
                                  _c_int(out.stride(0) if out is not None else N),
                                  _c_int(1 if (out is not None and out.dtype == torch.float32) else 0), _ptr(residual),
                                  _ptr(err), _stream()), "tc_linear")


def tc_swiglu(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out[M, I] = silu(x Wg^T) * (x Wu^T) with weight = [Wg; Wu] stacked [2I, K]; I a multiple of 64."""
    M, K = x.shape
    _check(library().vm_tc_swiglu(_ptr(x), _c_ll(x.stride(0)), _ptr(weight), _c_int(M), _c_int(out.shape[1]), _c_int(K),
                                  _ptr(_contig(out, "out")), _ptr(err), _stream()), "tc_swiglu")


def tc_qkv_rope(x: torch.Tensor, weight: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                block_table: torch.Tensor, inv_freq: Optional[torch.Tensor], rot_dim: int, k_pages: Optional[torch.Tensor],
                v_pages: Optional[torch.Tensor], H: int, Hkv: int, D: int, err: Optional[torch.Tensor] = None,
                pairing: int = 0) -> None:
    """Like skinny_qkv_rope for many rows: one head per tile, rotation and cache write in the epilogue. D 64 or 128."""
    M, K = x.shape
    n_pages = k_pages.shape[0] if k_pages is not None else 0
    _check(library().vm_tc_qkv_rope(_ptr(x), _c_ll(x.stride(0)), _ptr(weight), _c_int(M), _c_int(K), _ptr(_contig(q_out, "q_out")),
                                    _ptr(positions), _ptr(seq_of_token), _ptr(block_table), _c_int(block_table.shape[1]),
                                    _ptr(inv_freq), _c_int(rot_dim), _c_int(pairing), _ptr(k_pages), _ptr(v_pages), _c_int(H),
                                    _c_int(Hkv), _c_int(D), _c_int(n_pages), _ptr(err), _stream()), "tc_qkv_rope")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor,
           stream_id: torch.Tensor, step: torch.Tensor, out, step_add: int = 0) -> None:
    """One token per row of logits float32 [R, V]: greedy where temperature <= 0 or top_p <= 0, else
    temperature / nucleus sampling with a Philox draw keyed by (seed; stream_id, step + step_add) (all int64 [R]).
    `out`: an int32 device tensor, or an address from `host_device_pointer` (tokens written straight to the host)."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits are float32 rows")
    dst = _c_p(out) if isinstance(out, int) else _ptr(out)
    _check(library().vm_sample(_ptr(logits), _c_ll(logits.stride(0)), _c_int(R), _c_int(V), _ptr(temperature), _ptr(top_p),
                               _ptr(seed), _ptr(stream_id), _ptr(step), _c_ll(int(step_add)), dst, _stream()), "sample")


def host_device_pointer(pinned: torch.Tensor) -> int:
    """The address under which kernels reach the pinned host tensor `pinned`, or 0 if they cannot."""
    fn = library().vm_host_device_pointer
    fn.restype = ctypes.c_void_p
    return int(fn(_c_p(pinned.data_ptr())) or 0)


class CopyEvent:
    """An event that `upload` records behind a copy: `synchronize` returns when the copy has left the host buffer."""

    def __init__(self):
        lib = library()
        lib.vm_event_create.restype = ctypes.c_void_p
        self._destroy = lib.vm_event_destroy
        self._synchronize = lib.vm_event_synchronize
        self.handle = _c_p(lib.vm_event_create())
        if not self.handle.value:
            raise KernelError("could not create a CUDA event")

    def synchronize(self) -> None:
        _check(self._synchronize(self.handle), "event synchronize")

    def __del__(self):
        try:
            if self.handle.value:
                self._destroy(self.handle)
        except Exception:
            pass


def upload(dev: torch.Tensor, pinned: torch.Tensor, event: Optional[CopyEvent]) -> None:
    """dev <- pinned (the same number of bytes) on the current stream, `event` recorded behind the copy: one call into
    the runtime instead of a tensor copy and an event record."""
    global h2d_bytes
    nbytes = dev.numel() * dev.element_size()
    _check(library().vm_upload_record(_c_p(dev.data_ptr()), _c_p(pinned.data_ptr()), _c_ll(nbytes),
                                      event.handle if event is not None else _c_p(0), _stream()), "upload")
    h2d_bytes += nbytes


def decode_advance(sampled: torch.Tensor, tokens: torch.Tensor, positions: torch.Tensor, ctx_len: torch.Tensor,
                   draw_step: torch.Tensor, history: torch.Tensor, iteration: torch.Tensor) -> None:
    """After sampling a decode step: tokens <- sampled, positions/ctx_len/draw_step += 1, history[iteration] <- sampled,
    iteration += 1 (all on the device, so that several steps can be queued without the host)."""
    B = sampled.shape[0]
    _check(library().vm_decode_advance(_ptr(sampled), _ptr(tokens), _ptr(positions), _ptr(ctx_len), _ptr(draw_step),
                                       _ptr(history), _ptr(iteration), _c_int(B), _stream()), "decode_advance")


def require_cuda(device) -> torch.device:
    """The device an engine may run on, or a loud refusal."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise KernelLibraryError(f"device {dev} refused: this library has CUDA kernels only and no CPU fallback")
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device is available; this library has no CPU fallback")
    library()
    return dev
