"""Bookkeeping of the cache on the host: pages of tokens and slots of sequences.

The reference's cache is a dictionary of tensors that grows by allocate-and-copy at
every step and holds one rectangular batch (src/libllm/kv_cache.cc:27-67,
src/libllm/llama.cc:203-212).  Here storage is allocated once and handed out in pages
of ``page_size`` tokens; a sequence owns a slot and a list of pages per cache group, and
gives all of it back when it ends."""
from __future__ import annotations

from typing import List

from ..errors import CacheError


class PagePool:
    """Free list of page numbers with checks against loss and double use."""

    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError("a cache needs at least one page")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.n_pages - len(self._free)

    def take(self, n: int) -> List[int]:
        """n pages, or CacheError with nothing taken."""
        if n < 0:
            raise CacheError(f"cannot take {n} pages")
        if n > len(self._free):
            raise CacheError(f"the cache is full: {n} pages wanted, {len(self._free)} of "
                             f"{self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: List[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise CacheError(f"page {p} does not exist (pool of {self.n_pages})")
            if not self._held[p]:
                raise CacheError(f"page {p} is freed twice")
        if len(set(pages)) != len(pages):
            raise CacheError("a page is named twice in one release")
        for p in pages:
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, none both or neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.n_pages):
            if (p in free) == self._held[p]:
                raise CacheError(f"page {p} is {'both free and held' if p in free else 'lost'}")


class SlotTable:
    """Slots of sequences: lowest free slot first, so slots are used again at once."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError("a cache needs at least one slot")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._held = [False] * n_slots

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free slot: all {self.n_slots} sequences slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.n_slots:
            raise CacheError(f"slot {slot} does not exist ({self.n_slots} slots)")
        if not self._held[slot]:
            raise CacheError(f"slot {slot} is freed twice or was never taken")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._held[slot]

    def held(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._held[s]]
