"""Host-side bookkeeping of the cache: slots, pages and lengths.  No device code.

The reference keeps one dense ``[maxPos][kvDim]`` array per layer for its single
sequence (memory/kvcache.go:5-23) and resets it by setting ``Len = 0``
(memory/kvcache.go:25).  Here a *slot* stands for one sequence of a batch; its
keys and values live in fixed-size *pages* (64 positions) drawn from a pool per
group of layers, so the pool is sized by the number of tokens that live
requests hold, whatever their lengths.  A slot that is freed gives its pages
back; nothing is zeroed on reuse because attention never reads past a
sequence's length.

Groups: layers that keep all keys share the pool ``kind="full"``; layers that
keep a window of them have a pool of their own and give a page back as soon as
every position in it is behind the window of all queries still to come.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


class CacheError(RuntimeError):
    """Bookkeeping misuse or exhaustion (no free slot, no free page, double free)."""


class PagePool:
    """Free page numbers ``0 .. n_pages-1``; the lowest free page is handed out first.

    A prompt's pages are taken in one go, so lowest-first keeps a sequence's pages next to one another
    in memory however the pool was used before.
    """

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages))      # a heap: sorted lists are heaps
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("cache is full: no free page")
        p = heapq.heappop(self._free)
        self._held[p] = True
        return p

    def give(self, page: int) -> None:
        if not 0 <= page < self.n_pages or not self._held[page]:
            raise CacheError(f"page {page} given back but not held")
        self._held[page] = False
        heapq.heappush(self._free, page)


@dataclass
class GroupBook:
    name: str
    window: Optional[int]
    pool: PagePool
    # per slot: page of each logical page index, -1 where none is held
    tables: Dict[int, List[int]] = field(default_factory=dict)


class CacheBook:
    """Slots and their pages, per group.

    ``reserve(slot, n_new)`` makes room for ``n_new`` more positions and returns,
    per group, the table entries that changed (to be mirrored on the device);
    ``commit`` moves the length forward once the step has run.
    """

    def __init__(self, groups: Sequence[Tuple[str, Optional[int]]], n_pages: int, page_size: int, n_slots: int,
                 max_seq_len: int):
        if page_size <= 0 or n_slots <= 0 or max_seq_len <= 0:
            raise CacheError("page_size, n_slots and max_seq_len must be positive")
        self.page_size = page_size
        self.n_slots = n_slots
        self.max_seq_len = max_seq_len
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        self.groups: Dict[str, GroupBook] = {
            name: GroupBook(name, window, PagePool(n_pages)) for name, window in groups}
        self._free_slots: List[int] = list(range(n_slots - 1, -1, -1))
        self._len: Dict[int, int] = {}

    # ------------------------------------------------------------------ slots
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def live_slots(self) -> List[int]:
        return sorted(self._len)

    def take_slot(self) -> int:
        if not self._free_slots:
            raise CacheError("no free slot")
        s = self._free_slots.pop()
        self._len[s] = 0
        for g in self.groups.values():
            g.tables[s] = []
        return s

    def free_slot(self, slot: int) -> Dict[str, List[int]]:
        """Give the slot and its pages back; returns the pages released per group."""
        if slot not in self._len:
            raise CacheError(f"slot {slot} freed but not held")
        released: Dict[str, List[int]] = {}
        for g in self.groups.values():
            pages = [p for p in g.tables.pop(slot) if p >= 0]
            for p in pages:
                g.pool.give(p)
            released[g.name] = pages
        del self._len[slot]
        self._free_slots.append(slot)
        return released

    def length(self, slot: int) -> int:
        try:
            return self._len[slot]
        except KeyError:
            raise CacheError(f"slot {slot} is not held") from None

    # ------------------------------------------------------------------ pages
    def pages_needed(self, slot: int, n_new: int) -> int:
        """Pages the largest group would have to take for ``n_new`` more positions."""
        new_len = self.length(slot) + n_new
        need = (new_len + self.page_size - 1) // self.page_size
        return max(need - len(g.tables[slot]) for g in self.groups.values()) if self.groups else 0

    def reserve(self, slot: int, n_new: int) -> Dict[str, List[Tuple[int, int]]]:
        """Room for positions ``len .. len+n_new-1``; returns {group: [(page index, page)]} of changes."""
        cur = self.length(slot)
        if n_new <= 0:
            raise CacheError("a step must bring at least one token per sequence")
        new_len = cur + n_new
        if new_len > self.max_seq_len:
            raise CacheError(f"sequence would reach {new_len} positions; the limit is {self.max_seq_len}")
        need = (new_len + self.page_size - 1) // self.page_size
        changes: Dict[str, List[Tuple[int, int]]] = {}
        taken: List[Tuple[GroupBook, int]] = []
        try:
            for g in self.groups.values():
                table = g.tables[slot]
                ch: List[Tuple[int, int]] = []
                if g.window is not None:
                    # keys at t <= cur - window are behind every query from position cur on
                    dead_before = cur - g.window + 1  # first position still visible
                    for idx in range(min(len(table), max(0, dead_before) // self.page_size)):
                        if table[idx] >= 0:
                            g.pool.give(table[idx])
                            table[idx] = -1
                            ch.append((idx, -1))
                while len(table) < need:
                    p = g.pool.take()
                    taken.append((g, p))
                    table.append(p)
                    ch.append((len(table) - 1, p))
                changes[g.name] = ch
        except CacheError:
            for g, p in taken:  # leave the book as it was
                g.tables[slot].remove(p)
                g.pool.give(p)
            raise
        return changes

    def commit(self, slot: int, n_new: int) -> None:
        self._len[slot] = self.length(slot) + n_new

    def table(self, group: str, slot: int) -> List[int]:
        return list(self.groups[group].tables[slot])

    # ----------------------------------------------------------------- checks
    def check(self) -> None:
        """Invariant: every page is free or held by exactly one slot; same for slots."""
        for g in self.groups.values():
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {g.name}: a page is held twice")
            if len(held) + g.pool.n_free != g.pool.n_pages:
                raise CacheError(f"group {g.name}: {g.pool.n_pages - len(held) - g.pool.n_free} pages lost")
        if len(self._len) + len(self._free_slots) != self.n_slots:
            raise CacheError("a slot was lost")
        if set(self._len) & set(self._free_slots):
            raise CacheError("a slot is both held and free")
