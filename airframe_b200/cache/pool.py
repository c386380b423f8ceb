"""A pool of indices (cache slots, cache pages): each is either free or held
by exactly one owner.  Host-side bookkeeping only."""
from __future__ import annotations

import heapq


class CacheFull(RuntimeError):
    """No free slot or page is left."""


class PoolError(RuntimeError):
    """An index was given back that is not held (freed twice, or never taken)."""


class IndexPool:
    def __init__(self, size: int, what: str = "index"):
        if size < 0:
            raise ValueError(f"pool size must be >= 0, got {size}")
        self.size = size
        self.what = what
        self._free = list(range(size))      # a heap: the lowest free index goes out first
        self._held = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def is_held(self, i: int) -> bool:
        return i in self._held

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.size} are held)")
        i = heapq.heappop(self._free)
        self._held.add(i)
        return i

    def take_many(self, n: int) -> list:
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}s wanted, {len(self._free)} of {self.size} free")
        return [self.take() for _ in range(n)]

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise PoolError(f"{self.what} {i} is not held (freed twice or never taken)")
        self._held.remove(i)
        heapq.heappush(self._free, i)
