"""Free lists: pages of a cache group, and sequence slots."""
from __future__ import annotations

from typing import List

from ..errors import CacheError, CacheFull


class FreeList:
    """Integers 0..n-1, each either free or held.  Last freed, first reused, so a test
    that frees and allocates meets the same storage again at once."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise CacheError(f"cannot make a pool of {n} {what}s")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def free(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (pool of {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice (or was never allocated)")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Every index is free exactly once or held, never both, never lost."""
        if len(set(self._free)) != len(self._free):
            raise CacheError(f"a {self.what} sits in the free list twice")
        for i in self._free:
            if self._held[i]:
                raise CacheError(f"{self.what} {i} is both free and held")
        if sum(self._held) + len(self._free) != self.n:
            raise CacheError(f"a {self.what} is lost: {sum(self._held)} held + {len(self._free)} free != {self.n}")
