"""The cache: keys and values per layer run in pages, a slot per sequence, and beside it
fixed-size state per sequence.

Layer runs whose mixers have the same ``CacheNeed`` (kind, heads, head size, window)
form a group with storage and a page pool of its own: K and V of shape
[runs, pages, kv_heads, page_size, head_dim].  A sequence holds, per group, a list
mapping its logical pages (position // page_size) to pool pages; a "window" group gives
pages back as soon as every position in them has left the window."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import CacheError
from ..parts.base import CacheNeed, LayerCache, StateNeed
from .pages import PagePool, SlotTable


@dataclass
class CacheGroup:
    need: CacheNeed
    runs: List[int]                    # schedule entries that own storage here
    pool: PagePool
    k: Optional[torch.Tensor] = None   # [runs, pages, kv_heads, page_size, d]
    v: Optional[torch.Tensor] = None


@dataclass
class SequenceRecord:
    slot: int
    length: int = 0
    pages: List[List[int]] = field(default_factory=list)   # per group: logical page -> pool page, -1 released


class KVCache:
    def __init__(self, run_needs: Sequence[Optional[CacheNeed]], run_states: Sequence[Dict[str, StateNeed]],
                 capacity_tokens: int, dtype: torch.dtype, device, page_size: int = 64,
                 max_slots: Optional[int] = None, allocate: bool = True):
        """``run_needs[i]``: what schedule entry i wants cached (None: nothing of its own).
        ``capacity_tokens``: tokens all live sequences may hold together, each sequence's
        count rounded up to whole pages."""
        if page_size < 1 or capacity_tokens < 1:
            raise CacheError("cache capacity and page size must be positive")
        self.page_size = page_size
        self.n_pages = (capacity_tokens + page_size - 1) // page_size
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self.run_group: List[Optional[Tuple[int, int]]] = []      # entry -> (group, index in group)
        for i, need in enumerate(run_needs):
            if need is None:
                self.run_group.append(None)
                continue
            for g, grp in enumerate(self.groups):
                if grp.need == need:
                    break
            else:
                g = len(self.groups)
                self.groups.append(CacheGroup(need, [], PagePool(self.n_pages)))
            self.run_group.append((g, len(self.groups[g].runs)))
            self.groups[g].runs.append(i)
        if allocate:
            for grp in self.groups:
                shape = (len(grp.runs), self.n_pages, grp.need.n_kv_heads, page_size, grp.need.head_dim)
                grp.k = torch.zeros(shape, dtype=dtype, device=device)
                grp.v = torch.zeros(shape, dtype=dtype, device=device)
        self.slots = SlotTable(max_slots or self.n_pages)
        self.sequences: Dict[int, SequenceRecord] = {}
        # fixed-size state per sequence: entry -> name -> [slots, *shape]
        self.state: List[Dict[str, torch.Tensor]] = []
        for needs in run_states:
            self.state.append({n: torch.zeros((self.slots.n_slots,) + tuple(s.shape), dtype=s.dtype,
                                              device=device) for n, s in needs.items()} if allocate else {})

    # ---------------------------------------------------------------- sequences
    def open(self) -> int:
        slot = self.slots.take()
        self.sequences[slot] = SequenceRecord(slot, 0, [[] for _ in self.groups])
        for st in self.state:
            for t in st.values():
                t[slot].zero_()
        return slot

    def close(self, slot: int) -> None:
        rec = self.sequences.get(slot)
        if rec is None:
            raise CacheError(f"slot {slot} is not open (closed twice?)")
        for g, pages in enumerate(rec.pages):
            self.groups[g].pool.give_back([p for p in pages if p >= 0])
        del self.sequences[slot]
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        return self._rec(slot).length

    def _rec(self, slot: int) -> SequenceRecord:
        try:
            return self.sequences[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not open") from None

    def reserve(self, growth: Dict[int, int]) -> None:
        """Pages for every sequence of ``growth`` (slot -> new length).  Either all are
        granted or CacheError is raised and nothing has changed."""
        taken: List[Tuple[int, int, List[int]]] = []
        try:
            for slot, new_len in growth.items():
                rec = self._rec(slot)
                if new_len < rec.length:
                    raise CacheError(f"slot {slot}: a sequence cannot shrink ({rec.length} -> {new_len})")
                want = (new_len + self.page_size - 1) // self.page_size
                for g, grp in enumerate(self.groups):
                    missing = want - len(rec.pages[g])
                    if missing > 0:
                        pages = grp.pool.take(missing)
                        taken.append((slot, g, pages))
                        rec.pages[g].extend(pages)
        except CacheError:
            for slot, g, pages in reversed(taken):
                rec = self.sequences[slot]
                del rec.pages[g][len(rec.pages[g]) - len(pages):]
                self.groups[g].pool.give_back(pages)
            raise

    def commit(self, slot: int, new_len: int) -> None:
        """The sequence now holds ``new_len`` tokens; window groups drop pages no later
        query can see (a query at position p >= new_len sees keys > p - window)."""
        rec = self._rec(slot)
        rec.length = new_len
        for g, grp in enumerate(self.groups):
            if grp.need.kind == "window" and grp.need.window:
                first_needed = max(0, new_len - grp.need.window + 1)
                drop = []
                for lp in range(min(first_needed // self.page_size, len(rec.pages[g]))):
                    if rec.pages[g][lp] >= 0:
                        drop.append(rec.pages[g][lp])
                        rec.pages[g][lp] = -1
                if drop:
                    grp.pool.give_back(drop)

    def page_table(self, group: int, slots: Sequence[int], width: int) -> np.ndarray:
        """int32 [len(slots), width]; unused entries are 0 (never read: positions beyond
        a sequence's length are never asked for) and released ones -1."""
        out = np.zeros((len(slots), width), dtype=np.int32)
        for i, s in enumerate(slots):
            pages = self._rec(s).pages[group]
            if len(pages) > width:
                raise CacheError(f"slot {s} holds {len(pages)} pages, the step's table has {width}")
            out[i, :len(pages)] = pages
        return out

    def pages_needed(self, slot: int) -> int:
        return max((len(p) for p in self._rec(slot).pages), default=0)

    # ---------------------------------------------------------------- views for layer runs
    def layer_cache(self, entry: int, source: Optional[int], page_tables: List[torch.Tensor]) -> Optional[LayerCache]:
        """What schedule entry ``entry`` sees: its own storage, or that of ``source``."""
        owner = entry if source is None else source
        rg = self.run_group[owner]
        if rg is None:
            return None
        g, idx = rg
        grp = self.groups[g]
        return LayerCache(grp.k[idx], grp.v[idx], page_tables[g], self.page_size, writes=source is None, group=g)

    def check(self) -> None:
        """Host bookkeeping is consistent: no page lost, held twice or freed twice."""
        for g, grp in enumerate(self.groups):
            grp.pool.check()
            held = [p for rec in self.sequences.values() for p in rec.pages[g] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g}: a page belongs to two sequences")
            if len(held) != grp.pool.in_use:
                raise CacheError(f"group {g}: {grp.pool.in_use} pages are held, sequences own {len(held)}")
        if sorted(self.sequences) != self.slots.held():
            raise CacheError("open sequences and held slots differ")
