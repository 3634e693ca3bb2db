"""Host-side bookkeeping of the cache: sequence slots and key/value pages.

CodeClaper/tinyllama.c's prefix cache keeps a pool of physical token slots with a free
list and maps a request's logical positions to them (kvcache.h:26-31, kvcache.c:70-120).
Here the unit is coarser: a *slot* per live sequence (its fixed-size state and its row of
the block table) and *pages* of 64 positions for keys and values.  Both allocators refuse
to hand out what is held and to take back what is free, so a lost, doubly held or doubly
freed slot or page is an error at the call that causes it.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    pass


class IndexPool:
    """A pool of the integers 0..n-1; lowest free index first, so reuse is deterministic."""

    def __init__(self, n: int, what: str):
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))      # pop() yields the lowest index
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def held(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"out of {self.what}s: all {self.n} are held")
        i = self._free.pop()
        if self._held[i]:                                     # pragma: no cover - invariant
            raise CacheError(f"{self.what} {i} was on the free list while held")
        self._held[i] = True
        return i

    def free(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice (or was never held)")
        self._held[i] = False
        # keep the free list sorted descending so that alloc() returns the lowest index
        lo, hi = 0, len(self._free)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._free[mid] > i:
                lo = mid + 1
            else:
                hi = mid
        self._free.insert(lo, i)

    def check(self) -> None:
        """Every index is either held or free, exactly once."""
        if sorted(self._free + self.held()) != list(range(self.n)):
            raise CacheError(f"{self.what} pool is inconsistent: free={self._free} held={self.held()}")
