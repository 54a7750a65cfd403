"""Device storage of the cache and its mirror of the page tables.

Per group of run entries with equal needs, ONE allocation
``[entries, 2 (keys, values), pages, kv_heads, page_size, head_dim]`` in the
run's precision and one page table ``[slots, pages per sequence]`` (int32, -1
where no page is held).  The layout keeps one kv head's 64 positions of a page
contiguous, which is what the attention kernel streams.

The fixed-size per-sequence state lives beside it (:class:`StateArea`): one
tensor ``[slots, *shape]`` per run entry that asks for state, zeroed for a slot
when the slot is taken, in the spirit of the reference's ``SSMStateCache``
(memory/ssmstate.go:44-69), whose ``Reset`` runs together with the KV reset at
the start of a request (models/llm/generate.go:97-100).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheNeed, StateNeed
from .book import CacheBook, CacheError

PAGE_SIZE = 64


@dataclass
class CacheView:
    """What one run entry sees of the cache."""

    keys: torch.Tensor          # [pages, kv_heads, page_size, head_dim]
    values: torch.Tensor
    page_table: torch.Tensor    # [slots, pages per sequence] int32
    page_size: int
    writes: bool                # False when the entry reads another entry's cache


class StateArea:
    """Fixed-size per-sequence state, one tensor ``[slots, *shape]`` per entry that wants it."""

    def __init__(self, needs: Dict[int, StateNeed], n_slots: int, device: torch.device):
        self.tensors: Dict[int, torch.Tensor] = {
            e: torch.zeros((n_slots,) + tuple(n.shape), dtype=n.dtype, device=device) for e, n in needs.items()}

    def view(self, entry: int) -> Optional[torch.Tensor]:
        return self.tensors.get(entry)

    def reset_slot(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def snapshot(self, slots: Sequence[int]) -> Dict[int, torch.Tensor]:
        """Copies of the given slots' state (a run that must leave no trace restores them afterwards)."""
        idx = torch.tensor(list(slots), dtype=torch.int64)
        return {e: t[idx.to(t.device)].clone() for e, t in self.tensors.items()}

    def restore(self, slots: Sequence[int], saved: Dict[int, torch.Tensor]) -> None:
        idx = torch.tensor(list(slots), dtype=torch.int64)
        for e, t in self.tensors.items():
            t[idx.to(t.device)] = saved[e]

    def bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.tensors.values())


class KVCache:
    """Slots, pages and state for one model on one device.

    ``entry_needs[i]`` is what run entry ``i`` keeps (``None``: nothing, or it
    borrows: then ``borrows[i]`` names the lender).  ``max_tokens`` is the number
    of positions live sequences may hold in total, each sequence's count rounded
    up to a whole page.
    """

    def __init__(self, entry_needs: Sequence[Optional[CacheNeed]], borrows: Sequence[Optional[int]],
                 state_needs: Dict[int, StateNeed], max_tokens: int, max_seq_len: int, dtype: torch.dtype,
                 device: torch.device, page_size: int = PAGE_SIZE, n_slots: Optional[int] = None):
        self.page_size = page_size
        n_pages = max(1, (max_tokens + page_size - 1) // page_size)
        self.n_pages = n_pages
        self.n_slots = n_slots if n_slots is not None else n_pages
        self.max_seq_len = min(max_seq_len, n_pages * page_size)
        self.dtype = dtype
        self.device = device
        # group entries by (group name, heads, head_dim, window)
        keyed: Dict[Tuple, List[int]] = {}
        for i, need in enumerate(entry_needs):
            if need is None or borrows[i] is not None:
                continue
            keyed.setdefault((need.group, need.num_kv_heads, need.head_dim, need.window), []).append(i)
        names: Dict[Tuple, str] = {}
        for key in keyed:
            base = key[0]
            clash = [k for k in keyed if k[0] == base]
            names[key] = base if len(clash) == 1 else f"{base}/{key[1]}x{key[2]}w{key[3]}"
        self.book = CacheBook([(names[k], k[3]) for k in keyed], n_pages, page_size, self.n_slots, self.max_seq_len)
        self._no_window = all(k[3] is None for k in keyed)
        self.storage: Dict[str, torch.Tensor] = {}
        self.page_tables: Dict[str, torch.Tensor] = {}
        self._entry_place: Dict[int, Tuple[str, int]] = {}
        for key, entries in keyed.items():
            name = names[key]
            _, hkv, hd, _ = key
            self.storage[name] = torch.empty((len(entries), 2, n_pages, hkv, page_size, hd), dtype=dtype, device=device)
            self.page_tables[name] = torch.full((self.n_slots, self.book.max_pages_per_seq), -1, dtype=torch.int32,
                                                device=device)
            for j, e in enumerate(entries):
                self._entry_place[e] = (name, j)
        self._borrows = list(borrows)
        self.state = StateArea(state_needs, self.n_slots, device)
        self.poison_freed = bool(os.environ.get("DLGO_CACHE_POISON"))  # debug switch: unwritten cache reads as NaN
        if self.poison_freed:
            self.poison()

    # ------------------------------------------------------------------ views
    def view(self, entry: int) -> Optional[CacheView]:
        src = self._borrows[entry] if self._borrows[entry] is not None else entry
        place = self._entry_place.get(src)
        if place is None:
            return None
        name, j = place
        st = self.storage[name]
        return CacheView(st[j, 0], st[j, 1], self.page_tables[name], self.page_size, writes=src == entry)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.storage.values())

    # ------------------------------------------------------------------ slots
    def take_slot(self) -> int:
        slot = self.book.take_slot()
        self.state.reset_slot(slot)
        return slot

    def free_slot(self, slot: int) -> None:
        released = self.book.free_slot(slot)
        for pt in self.page_tables.values():
            pt[slot].fill_(-1)
        if self.poison_freed:
            for g, pages in released.items():
                if pages:
                    self.storage[g][:, :, torch.tensor(pages, device=self.device)] = float("nan")

    def length(self, slot: int) -> int:
        return self.book.length(slot)

    def reserve(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        """Room for each slot's new positions; mirrors changed table entries to the device."""
        if self._no_window and all(n == 1 for n in n_new):
            # decode steps mostly land inside the sequence's last page: nothing to take, give or mirror
            ps = self.page_size
            lengths = self.book._len
            try:
                if all(lengths[s] % ps and lengths[s] < self.max_seq_len for s in slots):
                    return
            except KeyError:
                pass                        # a slot that is not held: the full path reports it
        # all or nothing: a refused step takes no page, so the device tables never fall behind the book
        rows = self.book.reserve_batch(slots, n_new)
        for g, ch in rows.items():
            if not ch:
                continue
            pt = self.page_tables[g]
            idx = torch.tensor([s * pt.shape[1] + i for s, i, _ in ch], dtype=torch.int64)
            val = torch.tensor([p for _, _, p in ch], dtype=torch.int32)
            pt.view(-1).index_copy_(0, idx.to(self.device, non_blocking=True), val.to(self.device, non_blocking=True))

    def pages_short(self, slots: Sequence[int], n_new: Sequence[int]) -> Optional[str]:
        """``None`` if the pools hold the pages this step needs, else what is missing (nothing changes)."""
        return self.book.pages_short(slots, n_new)

    def commit(self, slots: Sequence[int], n_new: Sequence[int]) -> None:
        for slot, n in zip(slots, n_new):
            self.book.commit(slot, n)

    def poison(self, value: float = float("nan")) -> None:
        """Fill every page with ``value`` (tests: nothing unwritten may reach a result)."""
        self.poison_freed = True
        for st in self.storage.values():
            st.fill_(value)


__all__ = ["CacheError", "CacheView", "KVCache", "PAGE_SIZE", "StateArea"]
