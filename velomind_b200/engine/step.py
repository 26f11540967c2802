"""The step function: a batch of sequences, each bringing its next tokens; one pass from the cache.

The reference has two entry points for one sequence, `prefill(tokens)` and
`forward_step(token, pos)`, each of which builds, compiles and allocates a new
graph (examples/common/llama/llama_engine.cpp:333-393, :395-455).  Here one
function serves any batch: whole prompts of unequal lengths in one step, then
one token per sequence, or any other cut.  It runs only the tokens it is
given, packed without padding, reads and extends the cache in place, and
returns float32 logits at the wanted places.
"""
from __future__ import annotations

import gc

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.pages import PAGE_TOKENS, CacheError
from ..cache.store import SequenceCache
from ..kernels import ops
from .arena import Workspace
from .model import DecoderModel


@dataclass
class Entry:
    """One sequence's share of a step: its slot, its next tokens, and the places among these tokens
    (0-based) whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _bucket(n: int, fine_from: int = 512, fine_step: int = 512, floor: int = 8) -> int:
    """Capacity a count is rounded up to, so that few distinct buffer plans exist."""
    n = max(int(n), 1)
    if n <= fine_from:
        b = floor
        while b < n:
            b *= 2
        return b
    return -(-n // fine_step) * fine_step


GRAPHS_DEFAULT = True     # decode steps are replayed from CUDA graphs unless an Engine is told otherwise


def _host_buffer(n: int, dtype: torch.dtype) -> torch.Tensor:
    """Page-locked host memory, so that the copy to the device is asynchronous."""
    return torch.empty(n, dtype=dtype, pin_memory=True)


def _new_event():
    return ops.CopyEvent()


def _upload(dev: torch.Tensor, host: torch.Tensor, event) -> None:
    ops.upload(dev, host, event)


def _sync_stream() -> None:
    torch.cuda.current_stream().synchronize()


class Descriptors:
    """The integers that describe one step, laid out in one pinned host buffer and one device buffer of
    the same layout, so that a step costs one host-to-device copy."""

    def __init__(self, T: int, B: int, R: int, table_widths: Sequence[int], device):
        self.caps = (T, B, R, tuple(table_widths))
        fields = [("tokens", T), ("positions", T), ("seq_of_token", T), ("cu_tokens", B + 1), ("slots", B),
                  ("ctx_len", B), ("logit_rows", max(R, 1))]
        for g, w in enumerate(table_widths):
            fields.append((f"table{g}", B * w))
        self.offsets: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, n in fields:
            self.offsets[name] = (off, n)
            off += -(-n // 4) * 4          # 16-byte aligned fields
        self.total = off
        self.host = _host_buffer(off, torch.int32)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(off, dtype=torch.int32, device=device)
        self.copied = _new_event()
        self.used = False
        self.next_decode = None            # what a decode step described ahead of its tokens rests on (Engine._describe_next_decode)
        self.decode_slots = None           # the slots whose plain decode step the buffer describes (Engine._step_decode) ...
        self.decode_versions = None        # ... and the block tables' versions it was filled at

    def h(self, name: str) -> np.ndarray:
        off, n = self.offsets[name]
        return self.host_np[off: off + n]

    def d(self, name: str) -> torch.Tensor:
        off, n = self.offsets[name]
        return self.dev[off: off + n]

    def upload(self) -> None:
        _upload(self.dev, self.host, self.copied)
        self.used = True

    def wait_reusable(self) -> None:
        if self.used:
            self.copied.synchronize()


class StepContext:
    """What the parts see of a step: packed tokens and their places, the cache, scratch buffers.

    Device tensors (int32): tokens [T], positions [T] (place of each token in its sequence),
    seq_of_token [T] (index into the batch), cu_tokens [B+1] (token offsets of the sequences),
    slots [B] (cache slot of each sequence), ctx_len [B] (length after this step), logit_rows [R].
    Host copies of the same live in `host_*` numpy arrays.
    """

    def __init__(self, engine: "Engine", desc: Descriptors, T: int, B: int, R: int, table_widths: Sequence[int]):
        self.schedule = engine.model.plan.schedule      # (no reference to the engine itself: a kept context would tie a cycle)
        self.cache: SequenceCache = engine.cache
        self.ws: Workspace = engine.ws
        self.act_dtype: torch.dtype = engine.dtype
        self.err: torch.Tensor = engine.err
        self.T, self.B, self.R = T, B, R
        self.T_cap, self.B_cap, self.R_cap, _ = desc.caps
        self.desc = desc
        self.tokens = desc.d("tokens")[:T]
        self.positions = desc.d("positions")[:T]
        self.seq_of_token = desc.d("seq_of_token")[:T]
        self.cu_tokens = desc.d("cu_tokens")[:B + 1]
        self.slots = desc.d("slots")[:B]
        self.ctx_len = desc.d("ctx_len")[:B]
        self.logit_rows = desc.d("logit_rows")[:R]
        self.tables = [desc.d(f"table{g}").view(self.B_cap, w)[:B] for g, w in enumerate(table_widths)]
        self.host_positions = desc.h("positions")[:T]
        self.host_cu_tokens = desc.h("cu_tokens")[:B + 1]
        self.host_ctx_len = desc.h("ctx_len")[:B]
        self.host_slots = desc.h("slots")[:B]
        self.run: Optional[int] = None
        self.logits: Optional[torch.Tensor] = None
        # `capturing`: True while the step is recorded into a CUDA graph: no choice may depend on this step's lengths,
        # only on its shape (T, B, R, table widths)
        self.refresh()

    def refresh(self) -> None:
        """Re-read what depends on the values (not the shape) of the descriptors: a kept context serves a new step."""
        B, T = self.B, self.T
        self.max_ctx_len = int(self.host_ctx_len.max()) if B else 0
        self.max_new = int(np.diff(self.host_cu_tokens).max()) if B else 0
        self.one_token_each = (self.max_new == 1 and T == B)
        self.run = None
        self.capturing = False

    # ---- scratch
    def take_tokens(self, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A [T, cols] buffer (backed by capacity rows, so that the plan of the bucket fits every step in it)."""
        return self.ws.take((self.T_cap, cols), dtype)[: self.T]

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.ws.take(shape, dtype)

    # ---- the cache of the layer that is running
    def kv(self):
        """(k_pages, v_pages, block_table, owns) of the running schedule position: pages
        [n_pages, kv_heads, 64, head_dim], block_table int32 [B, width] (page of each 64-token block of each
        sequence of the batch; -1 where none), owns False when the run reads another run's cache."""
        g, layer = self.cache.where(self.run)
        group = self.cache.groups[g]
        k, v = group.layer(layer)
        owns = self.schedule[self.run].cache_of is None
        return k, v, self.tables[g], owns

    def state(self) -> Optional[torch.Tensor]:
        """The fixed-size float32 state [max_slots, n] of the running schedule position (index it with
        `ctx.slots`); None if the mixer asked for none.  Zeroed when a slot is opened."""
        return self.cache.state[self.run]


class Engine:
    """A model on one GPU with its cache: open/close sequence slots and step batches through the model."""

    def __init__(self, model: DecoderModel, max_tokens: int, max_slots: Optional[int] = None,
                 max_step_tokens: int = 8192, use_graphs: Optional[bool] = None,
                 fused_prefill_rows: Optional[int] = None, poison_freed: bool = False):
        if model.device is None:
            raise RuntimeError("the model has no weights bound; use load_model()")
        self.model = model
        self.device = ops.require_cuda(model.device)
        self.dtype = model.dtype
        self.vocab = model.plan.vocab_size
        self.max_step_tokens = int(max_step_tokens)
        self.fused_prefill_rows = fused_prefill_rows      # steps with at least this many tokens use the fused tcgen05 kernels
        # pages are whole: round the budget up
        max_tokens = -(-int(max_tokens) // PAGE_TOKENS) * PAGE_TOKENS
        self.cache = SequenceCache(model.cache_needs(), model.cache_shares(), max_tokens, model.plan.max_positions,
                                   self.dtype, self.device, max_slots)
        # (poison_freed: a debugging aid; every scratch buffer is filled with NaN the moment it is given back)
        self.ws = Workspace(self.device, poison=poison_freed)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._desc: Dict[Tuple, Descriptors] = {}
        self._logits: Optional[torch.Tensor] = None
        self._graphs: Dict[Tuple, "torch.cuda.CUDAGraph"] = {}
        self._next_decode: Optional[Descriptors] = None     # the buffer that holds a decode step described ahead
        self._last_decode_desc, self._last_decode_widths = None, None
        # (waiting for the device after every launch, a debugging switch of the kernel wrappers, cannot be recorded)
        self.use_graphs = (GRAPHS_DEFAULT if use_graphs is None else bool(use_graphs)) and model.graph_safe and not ops.SYNC_EVERY_OP
        self.graphs_captured = 0
        self._shape_seen: Dict[Tuple, int] = {}
        self._run_state = None
        self._contexts: Dict[Tuple, StepContext] = {}
        self.steps_run = 0

    # ---- slots
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ---- one step
    def step(self, entries: Sequence[Entry]) -> torch.Tensor:
        """Run the entries' tokens as one batch from the cache; return float32 logits [wanted, vocab] on the
        device, in the order of the entries and of each entry's `want`.  The tensor is valid until the next step."""
        entries = list(entries)
        if entries and len(entries) <= self.max_step_tokens and all(
                len(e.tokens) == 1 and len(e.want) == 1 and e.want[0] == 0 for e in entries):
            return self._step_decode(entries)
        self._validate(entries)
        n_rows = sum(len(e.want) for e in entries)
        logits = self._logits_buffer(n_rows)
        total = sum(len(e.tokens) for e in entries)
        if total <= self.max_step_tokens:
            chunks = [[(i, 0, len(e.tokens)) for i, e in enumerate(entries) if len(e.tokens)]]
        else:
            chunks = self._cut(entries)
        # rows come out in processing order (entry, then place); `order` maps them to the asked-for order
        produced: List[Tuple[int, int]] = []
        row0 = 0
        for chunk in chunks:
            if not chunk:
                continue
            rows_here = self._run_chunk(entries, chunk, logits, row0, produced)
            row0 += rows_here
        asked = [(i, int(w)) for i, e in enumerate(entries) for w in e.want]
        if produced != asked:
            index = {key: r for r, key in enumerate(produced)}
            perm = torch.tensor([index[k] for k in asked], dtype=torch.long, device=self.device)
            logits = logits[:n_rows].index_select(0, perm)
        self.steps_run += 1
        return logits[:n_rows]

    # ---- several decode steps without the host in between
    MAX_DECODE_RUN = 64

    def decode_many(self, slots: Sequence[int], last_tokens: Sequence[int], params, streams: Sequence[int],
                    draw_steps: Sequence[int], k: int) -> np.ndarray:
        """Feed `last_tokens` (one per slot) and decode `k` tokens for every slot: each step's sampled tokens are
        fed back ON THE DEVICE (no host round trip between steps).  `params[i]` are SamplingParams, `streams[i]`
        and `draw_steps[i]` the Philox stream and counter of sequence i's next draw.  Returns int32 [k, B]: the
        tokens sampled after each step.  The host decides afterwards where a sequence really ended; every slot's
        length has grown by k."""
        B = len(slots)
        k = int(k)
        if k < 1 or k > self.MAX_DECODE_RUN:
            raise ValueError(f"decode_many: k must be in 1..{self.MAX_DECODE_RUN}")
        entries = [Entry(s, [int(t)], [0]) for s, t in zip(slots, last_tokens)]
        self._validate(entries, extra=k - 1)
        st = self._decode_state(B)
        desc, T, _, R, widths, new_len, _ = self._describe(entries, [(i, 0, 1) for i in range(B)], reserve_extra=k - 1)
        hf, hi = st["host_f"].numpy(), st["host_i"].numpy()
        for r, p in enumerate(params):
            hf[0, r], hf[1, r] = p.temperature, p.top_p
            hi[0, r], hi[1, r], hi[2, r] = p.seed, streams[r], draw_steps[r]
        st["dev_f"].copy_(st["host_f"], non_blocking=True)
        st["dev_i"].copy_(st["host_i"], non_blocking=True)
        st["iteration"].zero_()
        ctx = self._context(desc, T, B, R, widths)
        logits = self._logits_buffer(B)
        ctx.logits = logits[:B]
        bucket = (desc.caps[0], desc.caps[1], desc.caps[2], True, self.fused_prefill_rows)

        def one_step():
            self._forward(ctx)
            ops.sample(ctx.logits, st["dev_f"][0, :B], st["dev_f"][1, :B], st["dev_i"][0, :B], st["dev_i"][1, :B],
                       st["dev_i"][2, :B], st["sampled"][:B])
            ops.decode_advance(st["sampled"][:B], ctx.tokens, ctx.positions, ctx.ctx_len, st["dev_i"][2, :B],
                               st["history"], st["iteration"])

        if self.use_graphs and self.ws.planned(bucket):
            key = ("run", bucket, (B, tuple(widths), logits.data_ptr(), st["sampled"].data_ptr()), self.ws.generation)
            graph = self._graphs.get(key)
            if graph is None:
                graph = self._record(ctx, bucket, key, one_step)
            for _ in range(k):
                graph.replay()
            ops.launch_count += k * graph.launches[0]
            ops.library_calls += k * graph.launches[1]
        else:
            for _ in range(k):
                ops.TC_FUSED_MIN_ROWS = self.fused_prefill_rows
                self.ws.begin(bucket)
                try:
                    one_step()
                except Exception:
                    self.ws.abort()
                    raise
                self.ws.end()
        st["history_host"][: k * B].copy_(st["history"][: k * B], non_blocking=True)
        _sync_stream()
        for i, e in enumerate(entries):
            self.cache.commit(e.slot, new_len[i] + k - 1)
        self.steps_run += k
        return st["history_host"].numpy()[: k * B].reshape(k, B).copy()

    def _decode_state(self, B: int):
        """Device buffers of the sampler and of the token feedback, sized for a batch of at least B."""
        st = self._run_state
        if st is None or st["cap"] < B:
            cap = _bucket(B, floor=8)
            st = {
                "cap": cap,
                "host_f": _host_buffer(2 * cap, torch.float32).view(2, cap),
                "host_i": _host_buffer(3 * cap, torch.int64).view(3, cap),
                "dev_f": torch.empty((2, cap), dtype=torch.float32, device=self.device),
                "dev_i": torch.empty((3, cap), dtype=torch.int64, device=self.device),
                "sampled": torch.empty(cap, dtype=torch.int32, device=self.device),
                "history": torch.empty(self.MAX_DECODE_RUN * cap, dtype=torch.int32, device=self.device),
                "history_host": _host_buffer(self.MAX_DECODE_RUN * cap, torch.int32),
                "iteration": torch.zeros(1, dtype=torch.int32, device=self.device),
            }
            self._run_state = st
        return st

    def raise_if_error(self) -> None:
        """Synchronise and raise if a kernel reported a fault of the step's descriptors (no page, bad id)."""
        code = int(self.err.item())
        if code:
            self.err.zero_()
            what = {1: "a token id outside the vocabulary", 2: "a cache write without a page",
                    3: "a cache read without a page", 4: "a tensor-core kernel gave up waiting on a barrier"}.get(code, f"code {code}")
            raise CacheError(f"a kernel reported {what}")

    # ---- internals
    def _validate(self, entries: Sequence[Entry], extra: int = 0) -> None:
        seen = set()
        need: Dict[int, int] = {}
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.is_held(e.slot):
                raise CacheError(f"slot {e.slot} is not open")
            n = len(e.tokens)
            if n == 0 and len(e.want):
                raise ValueError(f"slot {e.slot}: logits wanted but no tokens given")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab:
                    # the reference checks ids on the host before its embedding kernel too (src/executable.cpp:54-72)
                    raise ValueError(f"slot {e.slot}: token id {int(t)} outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"slot {e.slot}: wanted place {int(w)} outside the {n} tokens of this step")
            new_len = self.cache.length[e.slot] + n + extra
            if new_len > self.cache.max_positions:
                raise CacheError(f"slot {e.slot} would reach {new_len} tokens; the model's limit is {self.cache.max_positions}")
            need[e.slot] = new_len
        if not self.cache.can_hold(need):
            raise CacheError("out of cache pages for this step: the live sequences and the new tokens exceed max_tokens")

    def _cut(self, entries: Sequence[Entry]) -> List[List[Tuple[int, int, int]]]:
        """Cut a step that brings more than max_step_tokens into pieces (entry, first, last+1), in order."""
        chunks, cur, room = [], [], self.max_step_tokens
        for i, e in enumerate(entries):
            a, n = 0, len(e.tokens)
            while a < n:
                take = min(n - a, room)
                cur.append((i, a, a + take))
                a += take
                room -= take
                if room == 0:
                    chunks.append(cur)
                    cur, room = [], self.max_step_tokens
        if cur:
            chunks.append(cur)
        return chunks

    def _logits_buffer(self, rows: int) -> torch.Tensor:
        cap = _bucket(rows)
        if self._logits is None or self._logits.shape[0] < cap:
            self._logits = None
            self._logits = torch.empty((cap, self.vocab), dtype=torch.float32, device=self.device)
        return self._logits

    def _descriptors(self, T: int, B: int, R: int, widths: Sequence[int]) -> Descriptors:
        key = (_bucket(T), _bucket(B, floor=1), _bucket(R), tuple(widths))
        d = self._desc.get(key)
        if d is None:
            d = Descriptors(key[0], key[1], key[2], key[3], self.device)
            self._desc[key] = d
        return d

    def _forward(self, ctx: StepContext) -> None:
        self.model.forward(ctx)

    def _run_eager(self, ctx: StepContext, bucket) -> None:
        ops.TC_FUSED_MIN_ROWS = self.fused_prefill_rows
        self.ws.begin(bucket)
        try:
            self._forward(ctx)
        except Exception:
            self.ws.abort()
            raise
        self.ws.end()

    def _record(self, ctx: StepContext, bucket, key, body) -> "torch.cuda.CUDAGraph":
        """Record `body()` (the launches of one step) into a CUDA graph and keep it under `key`."""
        if len(self._graphs) >= 256:
            self._graphs.clear()
        ctx.capturing = True
        ops.TC_FUSED_MIN_ROWS = self.fused_prefill_rows
        graph = torch.cuda.CUDAGraph()
        torch.cuda.current_stream().synchronize()
        own, lib = ops.launch_count, ops.library_calls
        self.ws.begin(bucket)
        # the collector must not free another engine's graphs meanwhile: destroying a graph is not allowed while a
        # stream records, and ends the recording with an error
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                body()
        except Exception:
            self.ws.abort()
            raise
        finally:
            if collecting:
                gc.enable()
        self.ws.end()
        # what a replay launches: counted once here, added to the counters at every replay
        graph.launches = (ops.launch_count - own, ops.library_calls - lib)
        ops.launch_count, ops.library_calls = own, lib
        self._graphs[key] = graph
        self.graphs_captured += 1
        return graph

    def _replay_graph(self, ctx: StepContext, bucket, shape_key) -> "torch.cuda.CUDAGraph":
        """Steps are launch-bound (hundreds of small kernels): the kernels of a step are captured once per
        step shape into a CUDA graph and replayed.  Everything that changes from step to step (tokens,
        positions, lengths, block tables) lies in the descriptor buffer, which the graph reads.  A decode
        step's shape is (batch, table widths); any other step's shape also names each sequence's number of
        new tokens and the wanted rows, and is recorded only when it repeats."""
        key = (bucket, shape_key, self.ws.generation)
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._record(ctx, bucket, key, lambda: self._forward(ctx))
        graph.replay()
        ops.launch_count += graph.launches[0]
        ops.library_calls += graph.launches[1]
        return graph

    def _table_widths(self, slots: Sequence[int]) -> List[int]:
        """Per cache group, how wide the block tables of a batch of these slots are: the most blocks any of them holds,
        rounded up to a power of two (few distinct step shapes), at most the table's own width."""
        widths = []
        for g in self.cache.groups:
            need = max(1, max(g.blocks_end[slot] for slot in slots))
            w = 1
            while w < need:
                w *= 2
            widths.append(min(w, g.max_blocks))
        return widths

    def _describe(self, entries, chunk, reserve_extra: int = 0):
        """Reserve cache room for a chunk of a step and write its descriptors; returns (desc, T, B, R, widths,
        new lengths, wanted (entry, place) pairs).  `reserve_extra` tokens of room are reserved beyond the chunk's
        own (decode runs that queue several steps)."""
        cache = self.cache
        B = len(chunk)
        T = sum(b - a for _, a, b in chunk)
        new_len: List[int] = []
        for (i, a, b) in chunk:
            e = entries[i]
            cache.reserve(e.slot, cache.length[e.slot] + (b - a) + reserve_extra)
        widths = self._table_widths([entries[i].slot for i, _, _ in chunk])
        wanted_here = []
        for (i, a, b) in chunk:
            for w in sorted(int(x) for x in entries[i].want):
                if a <= w < b:
                    wanted_here.append((i, w))
        R = len(wanted_here)
        desc = self._descriptors(T, B, R, widths)
        desc.wait_reusable()
        desc.decode_slots = None
        desc.next_decode = None
        tok, pos, sot = desc.h("tokens"), desc.h("positions"), desc.h("seq_of_token")
        cu, slots, ctx_len, lrows = desc.h("cu_tokens"), desc.h("slots"), desc.h("ctx_len"), desc.h("logit_rows")
        if T == B:
            # one token per sequence (decode): everything in whole-array operations
            slot_ids = np.fromiter((entries[i].slot for i, _, _ in chunk), dtype=np.int64, count=B)
            base = np.fromiter((cache.length[int(x)] for x in slot_ids), dtype=np.int32, count=B)
            tok[:B] = np.fromiter((entries[i].tokens[a] for i, a, _ in chunk), dtype=np.int32, count=B)
            pos[:B] = base
            sot[:B] = np.arange(B, dtype=np.int32)
            cu[:B + 1] = np.arange(B + 1, dtype=np.int32)
            slots[:B] = slot_ids
            ctx_len[:B] = base + 1
            new_len = (base + 1).tolist()
            order = {i: s for s, (i, _, _) in enumerate(chunk)}
            for r, (i, w) in enumerate(wanted_here):
                lrows[r] = order[i]
            for g, group in enumerate(cache.groups):
                w = widths[g]
                desc.h(f"table{g}").reshape(desc.caps[1], w)[:B] = group.block_table[slot_ids, :w]
        else:
            t0 = 0
            cu[0] = 0
            start_of = {}
            for s, (i, a, b) in enumerate(chunk):
                e = entries[i]
                n = b - a
                base = cache.length[e.slot]
                tok[t0: t0 + n] = np.asarray(e.tokens[a:b], dtype=np.int32)
                pos[t0: t0 + n] = np.arange(base, base + n, dtype=np.int32)
                sot[t0: t0 + n] = s
                slots[s] = e.slot
                ctx_len[s] = base + n
                new_len.append(base + n)
                start_of[i] = t0 - a
                t0 += n
                cu[s + 1] = t0
            for r, (i, w) in enumerate(wanted_here):
                lrows[r] = start_of[i] + w
            for g, group in enumerate(cache.groups):
                w = widths[g]
                tab = desc.h(f"table{g}").reshape(desc.caps[1], w)
                for s, (i, _, _) in enumerate(chunk):
                    tab[s, :] = group.block_table[entries[i].slot, :w]
        desc.upload()
        return desc, T, B, R, widths, new_len, wanted_here

    def _context(self, desc, T: int, B: int, R: int, widths) -> StepContext:
        """The step's view of its descriptors.  Decode steps come in few shapes, and building the dozen tensor views
        costs as much host time as the rest of the step, so those contexts are kept and refreshed."""
        if T != B:
            return StepContext(self, desc, T, B, R, widths)
        key = (id(desc), T, B, R, tuple(widths))
        ctx = self._contexts.get(key)
        if ctx is None:
            if len(self._contexts) > 64:
                self._contexts.clear()
            ctx = StepContext(self, desc, T, B, R, widths)
            self._contexts[key] = ctx
        else:
            ctx.refresh()
        return ctx

    def _step_decode(self, entries: List[Entry]) -> torch.Tensor:
        """The common decode step (one new token per sequence, its logits wanted) with the host work of `step` cut to what
        this shape needs: the same checks, the same descriptors, no general bookkeeping.  Everything of the descriptors
        but the tokens is known before the tokens are: it is written for the NEXT step while the GPU runs this one
        (`_describe_next_decode`), and used if the same sequences then come again."""
        cache, B = self.cache, len(entries)
        lengths = cache.length
        slot_list = [e.slot for e in entries]
        toks = [int(e.tokens[0]) for e in entries]
        if len(set(slot_list)) != B:
            raise ValueError("a slot appears twice in one step")
        for slot, t in zip(slot_list, toks):
            if not 0 <= t < self.vocab:
                raise ValueError(f"slot {slot}: token id {t} outside the vocabulary of {self.vocab}")
        desc, self._next_decode = self._next_decode, None
        ahead = desc.next_decode if desc is not None else None
        graph = None
        if (ahead is not None and ahead[0] == slot_list and ahead[1] == [lengths[slot] for slot in slot_list]
                and ahead[2] == [g.version for g in cache.groups]):
            widths, graph = ahead[3], ahead[4]      # described ahead: nothing has touched these sequences or the pages since
        else:
            desc, widths = self._describe_decode(slot_list, True)
        desc.next_decode = None
        self._last_decode_desc, self._last_decode_widths = desc, widths
        desc.h("tokens")[:B] = toks
        desc.upload()
        logits = self._logits_buffer(B)
        made_for = (logits.data_ptr(), self.ws.generation, self.use_graphs, self.fused_prefill_rows)
        if graph is not None and graph[1] == made_for:
            # the graph that ran these sequences' last step: same shape, same buffers
            graph[0].replay()
            ops.launch_count += graph[0].launches[0]
            ops.library_calls += graph[0].launches[1]
        else:
            made = self._execute(desc, B, B, B, widths, logits, 0)
            graph = (made, made_for) if made is not None else None
        for slot in slot_list:
            cache.commit(slot, lengths[slot] + 1)
        self.steps_run += 1
        self._describe_next_decode(slot_list, graph)
        return logits[:B]

    def _describe_decode(self, slot_list: List[int], may_grow: bool):
        """Checks, cache room and descriptors (all but the tokens) of a decode step of the sequences in `slot_list`:
        (descriptors, table widths).  With `may_grow` False nothing is reserved and nothing raised: None comes back
        where the step needs a new page or is not allowed."""
        cache, B = self.cache, len(slot_list)
        lengths, held = cache.length, cache.slots.is_held
        grows = False
        for slot in slot_list:
            if not held(slot):
                if not may_grow:
                    return None
                raise CacheError(f"slot {slot} is not open")
            if lengths[slot] + 1 > cache.max_positions:
                if not may_grow:
                    return None
                raise CacheError(f"slot {slot} would reach {lengths[slot] + 1} tokens; the model's limit is {cache.max_positions}")
            grows = grows or lengths[slot] % PAGE_TOKENS == 0
        if grows:            # some sequence begins a new page: the general check and reservation
            if not may_grow:
                return None
            if not cache.can_hold({slot: lengths[slot] + 1 for slot in slot_list}):
                raise CacheError("out of cache pages for this step: the live sequences and the new tokens exceed max_tokens")
            for slot in slot_list:
                cache.reserve(slot, lengths[slot] + 1)
        widths = self._table_widths(slot_list)
        desc = self._descriptors(B, B, B, widths)
        desc.wait_reusable()
        desc.next_decode = None
        base = np.array([lengths[slot] for slot in slot_list], dtype=np.int32)
        desc.h("positions")[:B] = base
        desc.h("ctx_len")[:B] = base + 1
        versions = [g.version for g in cache.groups]
        if desc.decode_slots != slot_list or desc.decode_versions != versions:   # else the buffer still holds these rows and tables
            slot_ids = np.array(slot_list, dtype=np.int64)
            rows = np.arange(B + 1, dtype=np.int32)
            desc.h("seq_of_token")[:B] = rows[:B]
            desc.h("cu_tokens")[:B + 1] = rows
            desc.h("slots")[:B] = slot_ids
            desc.h("logit_rows")[:B] = rows[:B]
            for g, group in enumerate(cache.groups):
                w = widths[g]
                desc.h(f"table{g}").reshape(desc.caps[1], w)[:B] = group.block_table[slot_ids, :w]
            desc.decode_slots, desc.decode_versions = slot_list, versions
        return desc, widths

    def _describe_next_decode(self, slot_list: List[int], graph) -> None:
        """Called right after a decode step's launches, while the GPU works on them: the descriptors of the step that
        follows if the same sequences go on (all but its tokens).  Kept only with what it rests on (the slots, their
        lengths, the block tables' versions), so that any other use of the cache or of the buffer in between voids it."""
        described = self._describe_decode(slot_list, False)
        if described is None:
            return
        desc, widths = described
        lengths = self.cache.length
        if graph is not None and (desc is not self._last_decode_desc or widths != self._last_decode_widths):
            graph = None                   # the next step has another shape (a wider block table): another graph
        desc.next_decode = (slot_list, [lengths[slot] for slot in slot_list], [g.version for g in self.cache.groups], widths, graph)
        self._next_decode = desc

    def _run_chunk(self, entries, chunk, logits, row0, produced) -> int:
        cache = self.cache
        desc, T, B, R, widths, new_len, wanted_here = self._describe(entries, chunk)
        self._execute(desc, T, B, R, widths, logits, row0)
        for s, (i, a, b) in enumerate(chunk):
            cache.commit(entries[i].slot, new_len[s])
        produced.extend(wanted_here)
        return R

    def _execute(self, desc, T: int, B: int, R: int, widths, logits, row0: int):
        """Run the model on a described step: from its CUDA graph where there is one (which is returned), else part by
        part (None)."""
        ctx = self._context(desc, T, B, R, widths)
        ctx.logits = logits[row0: row0 + R]
        bucket = (desc.caps[0], desc.caps[1], desc.caps[2], ctx.one_token_each, self.fused_prefill_rows)   # decode steps take other scratch
        lens = tuple(int(x) for x in np.diff(ctx.host_cu_tokens)) if not ctx.one_token_each else ()
        shape_key = (T, B, R, tuple(widths), ctx.logits.data_ptr(), lens)
        use_graph = self.use_graphs and self.ws.planned(bucket)
        if use_graph and not ctx.one_token_each:
            # other steps (prompts) are recorded only when the very same shape comes a second time
            seen = self._shape_seen.get(shape_key, 0) + 1
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            self._shape_seen[shape_key] = seen
            use_graph = seen >= 2
        if use_graph:
            return self._replay_graph(ctx, bucket, shape_key)
        self._run_eager(ctx, bucket)
        return None
