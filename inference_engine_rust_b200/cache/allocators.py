"""Host-side bookkeeping of the cache: which slots and pages are held.

The reference has one cache per layer for a single sequence and "resets" by reallocating
(src/engine/session.rs:40-42, src/layers/attention.rs:27-39).  Here sequences come and go
in batches, so slots and pages are handed out and taken back; taking back twice, or
handing out what is held, is an error rather than silent corruption.
"""
from __future__ import annotations

from typing import Iterable, List, Set


class CacheError(RuntimeError):
    """Misuse of the cache: a slot or page freed twice, or not held."""


class CacheFull(CacheError):
    """No slot or page left (the reference's KVCacheFull, src/layers/attention.rs:55-59)."""


class IndexPool:
    """Hands out integers 0..n-1.  The most recently returned index is handed out next, so
    a slot that has just ended is the first to be used again."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"{what} pool size must be >= 0, got {n}")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held: Set[int] = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)

    def held(self) -> Set[int]:
        return set(self._held)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def alloc_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.alloc() for _ in range(k)]

    def free(self, i: int) -> None:
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never handed out)")
        self._held.remove(i)
        self._free.append(i)

    def free_many(self, items: Iterable[int]) -> None:
        for i in items:
            self.free(i)

    def check(self) -> None:
        """Every index is either free or held, exactly once."""
        if len(self._free) != len(set(self._free)):
            raise CacheError(f"{self.what} pool: an index is on the free list twice")
        if self._held & set(self._free):
            raise CacheError(f"{self.what} pool: an index is both held and free")
        if len(self._free) + len(self._held) != self.n:
            raise CacheError(f"{self.what} pool: {self.n - len(self._free) - len(self._held)} indices lost")
