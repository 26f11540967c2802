"""Bookkeeping of the cache on the host: sequence slots and pages of key/value storage.

The reference keeps ONE sequence whose key/value tensors are re-allocated and
copied on every decoded token (examples/common/llama/llama_engine.h:45-57,
llama_engine.cpp:442-446).  Here a batch of sequences each owns a slot; a slot
owns pages of `PAGE_TOKENS` tokens out of a fixed pool, so the memory is sized
by the number of tokens alive, not by slots x longest context.

Both allocators refuse misuse loudly (a page or slot freed twice, or one that
was never handed out), so that no page is lost or held twice.
"""
from __future__ import annotations

from typing import List

PAGE_TOKENS = 64


class CacheError(RuntimeError):
    """The cache was asked for more than it holds, or was misused."""


class FreeList:
    """Hands out integers 0..n-1; lowest free id first, so that a finished batch's ids are used again at once."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))  # pop() gives the lowest
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"out of {self.what}s: all {self.n} are in use")
        i = self._free.pop()
        assert not self._held[i], f"{self.what} {i} was on the free list while held"
        self._held[i] = True
        return i

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheError(f"out of {self.what}s: {k} wanted, {len(self._free)} of {self.n} free")
        return [self.take() for _ in range(k)]

    def give(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but was not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)
        # keep "lowest first": a sorted-descending list pops the lowest id
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Invariant: every id is either held or exactly once on the free list."""
        seen = [0] * self.n
        for i in self._free:
            seen[i] += 1
        for i in range(self.n):
            if seen[i] + (1 if self._held[i] else 0) != 1:
                raise CacheError(f"{self.what} {i}: on the free list {seen[i]} times, held={self._held[i]}")
