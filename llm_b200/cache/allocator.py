"""Bookkeeping of slots and pages, on the host.

A slot stands for one live sequence; a page holds the keys and values of 64
consecutive positions of one sequence for every layer of a group. Both come
from free lists and go back to them when the sequence ends; taking a slot or
page that is held, or returning one that is free, is an error, never silent.
"""
from __future__ import annotations

from ..errors import CacheFull, LlmError


class FreeList:
    """Integers 0 .. count-1, handed out lowest first and taken back."""

    def __init__(self, count: int, what: str):
        self.count = count
        self.what = what
        self._free = list(range(count - 1, -1, -1))     # pop() gives the lowest
        self._held = [False] * count

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.count - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.count} are held)")
        item = self._free.pop()
        if self._held[item]:
            raise LlmError(f"{self.what} {item} was on the free list while held")
        self._held[item] = True
        return item

    def give_back(self, item: int) -> None:
        if not 0 <= item < self.count:
            raise LlmError(f"{self.what} {item} does not exist")
        if not self._held[item]:
            raise LlmError(f"{self.what} {item} is freed twice")
        self._held[item] = False
        self._free.append(item)
        self._free.sort(reverse=True)

    def is_held(self, item: int) -> bool:
        return self._held[item]

    def check(self) -> None:
        """Every item is either free once or held, never both or neither."""
        seen = [0] * self.count
        for item in self._free:
            seen[item] += 1
        for item in range(self.count):
            if seen[item] + (1 if self._held[item] else 0) != 1:
                raise LlmError(f"{self.what} {item}: on the free list {seen[item]} times, "
                               f"held={self._held[item]}")
