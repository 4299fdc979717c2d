"""Host-side bookkeeping of the cache: which slots and which pages are held.  Pure Python, no
device access, so it is tested without a GPU.

ExiledOfCode/KuiperLLama has one sequence and one dense cache allocated for the full
context (kuiper/source/model/llama3.cpp:468-474); here a batch's sequences each take a slot
and grow page by page, and both are handed back and reused.
"""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """A misuse of the cache (a slot or page freed twice, none left, a request too long)."""


class FreeList:
    """Integers 0..n-1, handed out and taken back.  The one most recently returned is
    handed out first, so that a new sequence lands on storage that still holds an old
    sequence's contents (the case the tests want to see)."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))     # pop() yields 0 first
        self._held = [False] * n

    def available(self) -> int:
        return len(self._free)

    def held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def take_many(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheError(f"{count} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.take() for _ in range(count)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]


def pages_for(tokens: int, page: int) -> int:
    return (tokens + page - 1) // page
