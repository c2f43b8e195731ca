"""Host-side bookkeeping of the cache: which slots are in use and which pages they hold.

The reference keeps a fixed set of slots, each with a position counter, acquired for a
session and released at its end, bytes left in place for the next user
(src/kv_cache/kv_cache.cpp:85-134).  Here a slot holds a sequence of a batch; its storage
is a list of pages taken from a pool, so memory follows the tokens that are live, not
slots times the longest context.  Unlike the reference there is no stealing of a slot
that is in use: running out is an error before anything is launched.
"""
from __future__ import annotations

PAGE = 64          # positions a page of the cache holds


class CacheError(RuntimeError):
    """Out of slots or pages, or a slot used wrongly (freed twice, not held, over its length)."""


class PageAllocator:
    """A pool of ``n_pages`` page numbers.  A page is held by one owner at a time."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages - 1, -1, -1))      # pop() gives the lowest first
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheError(f"cache is full: {n} pages wanted, {len(self._free)} of "
                             f"{self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise CacheError(f"internal: page {p} handed out twice")
            self._held[p] = True
        return out

    def give_back(self, pages) -> None:
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise CacheError(f"page {p} given back but not held")
            self._held[p] = False
            self._free.append(p)


class SlotBook:
    """Slots 0..n_slots-1, each free or holding one sequence with its length."""

    def __init__(self, n_slots: int):
        self.n_slots = int(n_slots)
        self._free = list(range(self.n_slots - 1, -1, -1))
        self.in_use = [False] * self.n_slots
        self.length = [0] * self.n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise CacheError(f"no free slot: all {self.n_slots} slots hold live sequences")
        s = self._free.pop()
        if self.in_use[s]:
            raise CacheError(f"internal: slot {s} handed out twice")
        self.in_use[s] = True
        self.length[s] = 0
        return s

    def release(self, slot: int) -> None:
        self.check(slot)
        self.in_use[slot] = False
        self.length[slot] = 0
        self._free.append(slot)

    def check(self, slot: int) -> None:
        if not (0 <= slot < self.n_slots):
            raise CacheError(f"slot {slot} does not exist (slots 0..{self.n_slots - 1})")
        if not self.in_use[slot]:
            raise CacheError(f"slot {slot} is not held (released twice, or never acquired)")
