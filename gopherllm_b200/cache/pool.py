"""Host-side bookkeeping of the cache: which slots and pages are in use.

Pure Python, no device: the tests of "no slot lost, held twice or freed twice"
run on it directly.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """The cache cannot hold what was asked of it."""


class IdPool:
    """A fixed set of ids 0..n-1 handed out lowest-first and taken back."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))   # pop() gives the lowest
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} in use)")
        i = self._free.pop()
        assert not self._held[i], f"{self.what} {i} handed out twice"
        self._held[i] = True
        return i

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.take() for _ in range(k)]

    def give(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise ValueError(f"{self.what} {i} does not exist")
        if not self._held[i]:
            raise ValueError(f"{self.what} {i} is not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)
        # keep lowest-first order so reuse is deterministic
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Every id is either free or held, never both, never neither."""
        free = set(self._free)
        assert len(free) == len(self._free), f"a {self.what} is on the free list twice"
        for i in range(self.n):
            assert (i in free) != self._held[i], f"{self.what} {i} is lost or doubly owned"
