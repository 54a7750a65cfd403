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
        """Room for positions ``len .. len+n_new-1``; returns {group: [(page index, page)]} of changes.
        A refusal changes nothing."""
        return {g: [(idx, page) for _, idx, page in ch] for g, ch in self.reserve_batch([slot], [n_new]).items()}

    def reserve_batch(self, slots: Sequence[int], n_new: Sequence[int]) -> Dict[str, List[Tuple[int, int, int]]]:
        """:meth:`reserve` for all sequences of a step, all or nothing.

        Every check (slots held, lengths within the limit, pages of every pool) is made before the
        first page changes hands, so a refused step leaves the book exactly as it was: the reference
        likewise refuses a request before it touches its cache (models/llm/generate.go:85-90).
        Returns {group: [(slot, page index, page)]} of the entries that changed.
        """
        if len(slots) != len(n_new):
            raise CacheError(f"{len(slots)} slots for {len(n_new)} token counts")
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        ps = self.page_size
        plan: List[Tuple[int, int, int]] = []        # (slot, current length, pages needed afterwards)
        for slot, n in zip(slots, n_new):
            cur = self.length(slot)
            if n <= 0:
                raise CacheError("a step must bring at least one token per sequence")
            if cur + n > self.max_seq_len:
                raise CacheError(f"sequence would reach {cur + n} positions; the limit is {self.max_seq_len}")
            plan.append((slot, cur, (cur + n + ps - 1) // ps))
        for g in self.groups.values():
            takes = gives = 0
            for slot, cur, need in plan:
                table = g.tables[slot]
                takes += max(0, need - len(table))
                if g.window is not None:
                    dead = min(len(table), max(0, cur - g.window + 1) // ps)
                    gives += sum(1 for idx in range(dead) if table[idx] >= 0)
            if takes > g.pool.n_free + gives:
                raise CacheError(f"cache is full: group {g.name} needs {takes} more pages for this step, "
                                 f"{g.pool.n_free + gives} are free")
        changes: Dict[str, List[Tuple[int, int, int]]] = {g: [] for g in self.groups}
        # every give-back first, so that the pages a window released are there for the takes
        for g in self.groups.values():
            if g.window is None:
                continue
            for slot, cur, _ in plan:
                table = g.tables[slot]
                for idx in range(min(len(table), max(0, cur - g.window + 1) // ps)):
                    if table[idx] >= 0:
                        g.pool.give(table[idx])
                        table[idx] = -1
                        changes[g.name].append((slot, idx, -1))
        for g in self.groups.values():
            for slot, _, need in plan:
                table = g.tables[slot]
                while len(table) < need:
                    table.append(g.pool.take())
                    changes[g.name].append((slot, len(table) - 1, table[-1]))
        return changes

    def pages_short(self, slots: Sequence[int], n_new: Sequence[int]) -> Optional[str]:
        """``None`` if the pools hold the pages this step needs, else a sentence that says what is missing.
        Slots must be held and distinct; nothing changes."""
        ps = self.page_size
        for g in self.groups.values():
            takes = gives = 0
            for slot, n in zip(slots, n_new):
                cur = self.length(slot)
                table = g.tables[slot]
                takes += max(0, (cur + n + ps - 1) // ps - len(table))
                if g.window is not None:
                    dead = min(len(table), max(0, cur - g.window + 1) // ps)
                    gives += sum(1 for idx in range(dead) if table[idx] >= 0)
            if takes > g.pool.n_free + gives:
                return (f"the cache is full: group {g.name} needs {takes} more pages for this step, "
                        f"{g.pool.n_free + gives} are free")
        return None

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
