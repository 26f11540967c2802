"""Key/value storage for groups of layers, and fixed-size per-sequence state beside it.

A mixer declares what it needs to remember per sequence as a `CacheNeed`:
keys and values of all earlier tokens, of a window of them, nothing, and/or a
fixed number of float32 values (the place for a recurrent or convolutional
state).  Layers with equal needs share a `CacheGroup`: one pool of pages and
one block table per sequence slot; groups with different needs (all keys /
a window) have storage and bookkeeping of their own.

Page layout on the device: `k[layer, page, kv_head, token_in_page, head_dim]`
(the same for `v`): the 64 x head_dim tile of one kv head is contiguous.
Keys are stored after the position encoding, as the reference caches them
(examples/common/llama/llama_graph.cpp:210-215).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import PAGE_TOKENS, CacheError, FreeList


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer keeps per sequence."""
    kind: str = "none"            # "all": every earlier key/value; "window": the last `window`; "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_floats: int = 0         # fixed-size float32 state per sequence (0: none)

    def group_key(self) -> Tuple:
        return (self.kind, self.kv_heads, self.head_dim, self.window)


class CacheGroup:
    """Pages and block tables for the layers that share one `CacheNeed`."""

    def __init__(self, need: CacheNeed, n_layers: int, n_pages: int, max_slots: int, max_blocks: int,
                 dtype: torch.dtype, device):
        if need.kind not in ("all", "window"):
            raise CacheError(f"a cache group holds keys and values; kind {need.kind!r} needs none")
        if need.kind == "window" and need.window <= 0:
            raise CacheError("a window group needs window > 0")
        self.need = need
        self.n_layers = n_layers
        self.n_pages = n_pages
        self.max_blocks = max_blocks
        self.pages = FreeList(n_pages, "cache page")
        self.block_table = np.full((max_slots, max_blocks), -1, dtype=np.int32)
        self.blocks_end = [0] * max_slots      # logical blocks [blocks_begin, blocks_end) hold a page
        self.version = 0                       # grows whenever an entry of the block table changes
        self.blocks_begin = [0] * max_slots
        shape = (n_layers, n_pages, need.kv_heads, PAGE_TOKENS, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, -(-new_len // PAGE_TOKENS) - self.blocks_end[slot])

    def ensure(self, slot: int, new_len: int) -> None:
        """Give `slot` pages so that tokens [0, new_len) have a place."""
        want = -(-new_len // PAGE_TOKENS)
        if want > self.max_blocks:
            raise CacheError(f"a sequence of {new_len} tokens needs {want} blocks; the table holds {self.max_blocks}")
        k = want - self.blocks_end[slot]
        if k <= 0:
            return
        ids = self.pages.take_many(k)
        for j, pg in enumerate(ids):
            self.block_table[slot, self.blocks_end[slot] + j] = pg
        self.blocks_end[slot] = want
        self.version += 1

    def trim(self, slot: int, length: int) -> None:
        """After a step: a window group gives back the pages no later query can reach."""
        if self.need.kind != "window":
            return
        # the next query sits at position `length` or later and sees keys at positions > length - window
        first_needed = max(0, length - self.need.window + 1)
        b = self.blocks_begin[slot]
        while b < self.blocks_end[slot] and (b + 1) * PAGE_TOKENS <= first_needed:
            self.pages.give(int(self.block_table[slot, b]))
            self.block_table[slot, b] = -1
            b += 1
            self.version += 1
        self.blocks_begin[slot] = b

    def release(self, slot: int) -> None:
        for b in range(self.blocks_begin[slot], self.blocks_end[slot]):
            self.pages.give(int(self.block_table[slot, b]))
            self.block_table[slot, b] = -1
        self.blocks_begin[slot] = 0
        self.blocks_end[slot] = 0
        self.version += 1

    def layer(self, i: int):
        return self.k[i], self.v[i]


class SequenceCache:
    """Slots for sequences; for each slot its length, its pages in every group and its fixed-size state.

    `needs[i]` is the CacheNeed of schedule position i (None where the run reads another run's cache).
    `max_tokens` counts tokens of live sequences, each sequence rounded up to a multiple of the page size.
    """

    def __init__(self, needs: Sequence[Optional[CacheNeed]], shares: Sequence[Optional[int]], max_tokens: int,
                 max_positions: int, dtype: torch.dtype, device, max_slots: Optional[int] = None):
        if max_tokens < PAGE_TOKENS:
            raise CacheError(f"max_tokens {max_tokens} is less than one page of {PAGE_TOKENS} tokens")
        self.n_pages = max_tokens // PAGE_TOKENS
        self.max_positions = max_positions
        self.max_blocks = -(-max_positions // PAGE_TOKENS)
        self.max_slots = int(max_slots) if max_slots else min(self.n_pages, 4096)
        self.slots = FreeList(self.max_slots, "sequence slot")
        self.length = [0] * self.max_slots
        self.dtype = dtype
        self.device = device
        self.groups: List[CacheGroup] = []
        self._where: List[Optional[Tuple[int, int]]] = []   # schedule position -> (group, layer in group)
        by_key: Dict[Tuple, List[int]] = {}
        for i, need in enumerate(needs):
            if need is not None and need.kind != "none":
                by_key.setdefault(need.group_key(), []).append(i)
        slots_of: Dict[int, Tuple[int, int]] = {}
        for key, runs in by_key.items():
            g = CacheGroup(needs[runs[0]], len(runs), self.n_pages, self.max_slots, self.max_blocks, dtype, device)
            for j, run in enumerate(runs):
                slots_of[run] = (len(self.groups), j)
            self.groups.append(g)
        for i, need in enumerate(needs):
            owner = shares[i] if shares[i] is not None else i
            self._where.append(slots_of.get(owner))
        # fixed-size state: one float32 area [max_slots, n] for every run that asks for one
        self.state: List[Optional[torch.Tensor]] = []
        for i, need in enumerate(needs):
            n = need.state_floats if (need is not None and shares[i] is None) else 0
            self.state.append(torch.zeros((self.max_slots, n), dtype=torch.float32, device=device) if n else None)
        for i, owner in enumerate(shares):
            if owner is not None:
                self.state[i] = self.state[owner]

    # ---- slots
    def open(self) -> int:
        slot = self.slots.take()
        self.length[slot] = 0
        for st in self.state:
            if st is not None:
                st[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"sequence slot {slot} is closed but was not open")
        for g in self.groups:
            g.release(slot)
        self.length[slot] = 0
        self.slots.give(slot)

    def can_hold(self, new_lengths: Dict[int, int]) -> bool:
        for g in self.groups:
            if sum(g.pages_needed(s, n) for s, n in new_lengths.items()) > g.pages.free_count:
                return False
        return True

    def reserve(self, slot: int, new_len: int) -> None:
        """Make room for tokens [length, new_len) of `slot` in every group, or raise CacheError and change nothing."""
        if not self.slots.is_held(slot):
            raise CacheError(f"sequence slot {slot} is not open")
        if new_len > self.max_positions:
            raise CacheError(f"sequence would reach {new_len} tokens; the model's limit is {self.max_positions}")
        for g in self.groups:
            if g.pages_needed(slot, new_len) > g.pages.free_count:
                raise CacheError(
                    f"out of cache pages: slot {slot} needs {g.pages_needed(slot, new_len)} more pages of "
                    f"{PAGE_TOKENS} tokens, {g.pages.free_count} of {g.n_pages} free")
        for g in self.groups:
            g.ensure(slot, new_len)

    def commit(self, slot: int, new_len: int) -> None:
        self.length[slot] = new_len
        for g in self.groups:
            g.trim(slot, new_len)

    # ---- views for the step function
    def where(self, run: int) -> Optional[Tuple[int, int]]:
        return self._where[run]

    def tokens_held(self) -> int:
        """Tokens of live sequences, each rounded up to whole pages (what `max_tokens` bounds)."""
        return max((g.pages.held_count for g in self.groups), default=0) * PAGE_TOKENS

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            held = set()
            for s in range(self.max_slots):
                for b in range(g.max_blocks):
                    pg = int(g.block_table[s, b])
                    inside = g.blocks_begin[s] <= b < g.blocks_end[s]
                    if (pg >= 0) != inside:
                        raise CacheError(f"slot {s} block {b}: page {pg} but live range is [{g.blocks_begin[s]}, {g.blocks_end[s]})")
                    if pg >= 0:
                        if pg in held:
                            raise CacheError(f"cache page {pg} is held twice")
                        if not self.slots.is_held(s):
                            raise CacheError(f"cache page {pg} belongs to closed slot {s}")
                        held.add(pg)
            if len(held) != g.pages.held_count:
                raise CacheError(f"{g.pages.held_count} pages are marked held but block tables name {len(held)}")
