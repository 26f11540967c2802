"""Device time per kind of operation, behind a switch: what the reference gets from its per-run timers
(examples/common/llama/llama_engine.cpp:630,657-664; benchmarks/benchmark_runner.cpp:139-158), split by operation.

    with OpTimes() as times:
        engine.step(...)            # an engine made with use_graphs=False: a replayed graph passes by the wrappers
    print(times.table())

While the block runs, every public function of `kernels.ops` that launches work is bracketed by two CUDA events on
the current stream; leaving the block waits for the device once and adds the intervals up per function name.  The
events serialise nothing, but the intervals of kernels that overlap under programmatic dependent launch overlap too:
the sum over operations can exceed the step's time.  Nothing is wrapped outside the block.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

from . import ops

# the functions of `ops` that launch device work (bookkeeping helpers such as decode_splits are left alone)
TIMED = ("embed_gather", "add_rmsnorm", "residual_add", "swiglu", "convert", "rope_kv_write", "attention_generic",
         "attention_prefill_bf16", "attention_prefill_tc_bf16", "attention_decode_bf16", "linear", "skinny_linear",
         "skinny_swiglu", "skinny_qkv_rope", "tc_linear", "tc_swiglu", "tc_qkv_rope", "sample", "decode_advance",
         "upload")


def _cuda_event():
    import torch
    return torch.cuda.Event(enable_timing=True)


class OpTimes:
    def __init__(self, names: Optional[Tuple[str, ...]] = None, event: Callable = _cuda_event, module=ops):
        self.names = tuple(n for n in (names or TIMED) if hasattr(module, n))
        self._event, self._module = event, module
        self._saved: Dict[str, Callable] = {}
        self._pairs: List[Tuple[str, object, object]] = []
        self.ms: Dict[str, float] = {}
        self.calls: Dict[str, int] = {}

    def __enter__(self) -> "OpTimes":
        for name in self.names:
            fn = getattr(self._module, name)
            self._saved[name] = fn
            setattr(self._module, name, self._timed(name, fn))
        return self

    def _timed(self, name: str, fn: Callable) -> Callable:
        def call(*args, **kwargs):
            a, b = self._event(), self._event()
            a.record()
            try:
                return fn(*args, **kwargs)
            finally:
                b.record()
                self._pairs.append((name, a, b))
        call.__name__ = getattr(fn, "__name__", name)
        call.__doc__ = fn.__doc__
        return call

    def __exit__(self, *exc) -> None:
        for name, fn in self._saved.items():
            setattr(self._module, name, fn)
        self._saved = {}
        for name, a, b in self._pairs:
            b.synchronize()
            self.ms[name] = self.ms.get(name, 0.0) + float(a.elapsed_time(b))
            self.calls[name] = self.calls.get(name, 0) + 1
        self._pairs = []

    def table(self) -> str:
        total = sum(self.ms.values()) or 1.0
        rows = sorted(self.ms.items(), key=lambda kv: -kv[1])
        lines = [f"{'operation':<28}{'calls':>8}{'ms':>12}{'share':>9}"]
        for name, ms in rows:
            lines.append(f"{name:<28}{self.calls[name]:>8}{ms:>12.3f}{100.0 * ms / total:>8.1f}%")
        return "\n".join(lines)
