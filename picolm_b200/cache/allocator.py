"""Host-side bookkeeping of the cache: which sequence slots and which pages
are in use.  Pure Python, no device.  Every misuse (taking from an empty pool,
freeing twice, freeing what was never given) raises, so that a slot or a page can
never be lost or held twice.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """The cache cannot hold what was asked of it."""


class IndexPool:
    """A pool of the integers [first, first + count), handed out lowest first."""

    def __init__(self, count: int, first: int = 0, what: str = "index"):
        if count < 0:
            raise ValueError("count must not be negative")
        self.what = what
        self.first, self.count = first, count
        self._free: List[int] = list(range(first + count - 1, first - 1, -1))   # stack, lowest on top
        self._used = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return len(self._used)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what}: all {self.count} are in use")
        i = self._free.pop()
        self._used.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._used:
            if self.first <= i < self.first + self.count:
                raise RuntimeError(f"{self.what} {i} was freed twice")
            raise RuntimeError(f"{self.what} {i} does not belong to this pool")
        self._used.remove(i)
        self._free.append(i)

    def holds(self, i: int) -> bool:
        return i in self._used

    def check(self) -> None:
        """Every index is either free or used, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self.what} is in the free list twice")
        if free & self._used:
            raise AssertionError(f"a {self.what} is both free and used")
        if free | self._used != set(range(self.first, self.first + self.count)):
            raise AssertionError(f"a {self.what} was lost")
