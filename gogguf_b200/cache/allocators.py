"""Free-list allocators for sequence slots and cache pages (host side, no GPU).

A slot or page is held by exactly one owner at a time: taking from an empty list,
giving back what is not held, or giving back twice raises `CacheError`.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """Misuse or exhaustion of the cache: no free slot or page, double free, unknown slot."""


class CacheFull(CacheError):
    """Not enough free slots or pages for the request."""


class FreeList:
    """Ids 0..n-1; last freed is first reused, so reuse shows up early in tests."""

    def __init__(self, n: int, what: str = "slot"):
        if n < 0:
            raise ValueError(f"number of {what}s must be >= 0")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted but only {len(self._free)} of {self.n} are free")
        return [self.take() for _ in range(k)]

    def give(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)

    def check(self) -> None:
        """Invariant: every id is either free once or held, never both."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.n):
            if self._held[i] == (i in seen):
                raise CacheError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")
