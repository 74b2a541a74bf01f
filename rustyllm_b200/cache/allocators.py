"""Host-side bookkeeping of the cache: which slots and which pages are in use.

A *slot* is one sequence's place in the cache (its length, its row of every page
table, its state area).  A *page* holds the keys and values of ``page_size``
consecutive positions for all layers of one storage group.  Both allocators are
strict: handing out something that is held, or taking back something that is not,
raises instead of corrupting the cache.  In the reference a cache belongs to one
generation or one session (src/model.rs:1328-1349, src/session.rs:86-143); slots
that are given back and used again by the next batch are this library's own.
"""
from __future__ import annotations

from typing import Iterable, List


class CacheFull(RuntimeError):
    """Not enough free slots or pages for what was asked."""


class CacheMisuse(RuntimeError):
    """A slot or page was freed twice, or used while not held."""


class FreeList:
    """Ids 0..n-1, each either free or held.  Lowest free id first, so runs are
    reproducible and freed ids are reused at once (which tests rely on to show that
    stale contents of a reused slot or page are never read)."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"number of {what}s must be >= 0")
        self._n = n
        self._what = what
        self._held = [False] * n
        self._free = list(range(n - 1, -1, -1))  # stack; lowest id on top
        self._dirty = False

    @property
    def capacity(self) -> int:
        return self._n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self._n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self._n and self._held[i]

    def take(self, count: int = 1) -> List[int]:
        if count < 0:
            raise ValueError("count must be >= 0")
        if count > len(self._free):
            raise CacheFull(f"{count} {self._what}(s) wanted, {len(self._free)} of {self._n} free")
        if self._dirty:
            self._free.sort(reverse=True)
            self._dirty = False
        out = []
        for _ in range(count):
            i = self._free.pop()
            self._held[i] = True
            out.append(i)
        return out

    def give_back(self, ids: Iterable[int]) -> None:
        ids = list(ids)
        for i in ids:
            if not (0 <= i < self._n):
                raise CacheMisuse(f"{self._what} {i} does not exist (0..{self._n - 1})")
            if not self._held[i]:
                raise CacheMisuse(f"{self._what} {i} is given back but is not held (freed twice?)")
            self._held[i] = False
            self._free.append(i)
        if ids:
            self._dirty = True

    def check(self) -> None:
        """Invariant: every id is exactly one of held / free."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheMisuse(f"a {self._what} is on the free list twice")
        for i in range(self._n):
            if self._held[i] == (i in free):
                raise CacheMisuse(f"{self._what} {i} is {'both held and free' if self._held[i] else 'lost'}")
