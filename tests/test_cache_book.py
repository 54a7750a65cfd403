"""Cache bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from dlgo_b200.cache import CacheBook, CacheError, PagePool


def test_page_pool_take_give():
    p = PagePool(3)
    got = {p.take(), p.take(), p.take()}
    assert got == {0, 1, 2} and p.n_free == 0
    with pytest.raises(CacheError, match="full"):
        p.take()
    p.give(1)
    with pytest.raises(CacheError, match="not held"):
        p.give(1)
    with pytest.raises(CacheError):
        p.give(7)
    assert p.take() == 1


def test_page_pool_hands_out_the_lowest_free_page():
    # whatever order pages came back in, a prompt's pages are taken next to one another again
    p = PagePool(8)
    held = [p.take() for _ in range(8)]
    assert held == list(range(8))
    for page in (5, 2, 7, 3):
        p.give(page)
    assert [p.take(), p.take(), p.take(), p.take()] == [2, 3, 5, 7]
    b = CacheBook([("full", None)], n_pages=8, page_size=64, n_slots=4, max_seq_len=512)
    s0, s1 = b.take_slot(), b.take_slot()
    b.reserve(s0, 130); b.commit(s0, 130)
    b.reserve(s1, 100); b.commit(s1, 100)
    b.free_slot(s0)
    s2 = b.take_slot()
    b.reserve(s2, 200); b.commit(s2, 200)
    assert b.table("full", s2) == [0, 1, 2, 5]
    b.check()


def test_slots_and_pages_follow_lengths():
    b = CacheBook([("full", None)], n_pages=4, page_size=64, n_slots=3, max_seq_len=256)
    s = b.take_slot()
    ch = b.reserve(s, 5)
    assert ch["full"] == [(0, b.table("full", s)[0])]
    b.commit(s, 5)
    assert b.reserve(s, 59)["full"] == []            # still inside the first page
    b.commit(s, 59)
    assert len(b.reserve(s, 1)["full"]) == 1         # position 64 opens the second page
    b.commit(s, 1)
    assert b.length(s) == 65 and len(b.table("full", s)) == 2
    b.check()
    with pytest.raises(CacheError, match="limit"):
        b.reserve(s, 200)
    released = b.free_slot(s)
    assert len(released["full"]) == 2 and b.groups["full"].pool.n_free == 4
    with pytest.raises(CacheError, match="not held"):
        b.free_slot(s)
    with pytest.raises(CacheError, match="not held"):
        b.length(s)
    b.check()


def test_exhaustion_leaves_the_book_consistent():
    b = CacheBook([("full", None)], n_pages=2, page_size=64, n_slots=2, max_seq_len=1024)
    s0, s1 = b.take_slot(), b.take_slot()
    with pytest.raises(CacheError, match="no free slot"):
        b.take_slot()
    b.reserve(s0, 64)
    b.commit(s0, 64)
    with pytest.raises(CacheError, match="full"):
        b.reserve(s1, 129)          # needs 3 pages, 1 is free
    b.check()
    assert b.groups["full"].pool.n_free == 1 and b.table("full", s1) == []
    b.reserve(s1, 10)
    b.check()


def test_window_group_gives_pages_back_and_keeps_a_pool_of_its_own():
    b = CacheBook([("full", None), ("win", 100)], n_pages=8, page_size=64, n_slots=2, max_seq_len=512)
    s = b.take_slot()
    b.reserve(s, 300)
    b.commit(s, 300)
    assert len(b.table("full", s)) == 5 and len(b.table("win", s)) == 5
    ch = b.reserve(s, 1)     # queries from position 300 on see keys > 200: pages 0..2 are behind the window
    assert sorted(i for i, p in ch["win"] if p == -1) == [0, 1, 2]
    assert b.table("win", s)[:3] == [-1, -1, -1] and all(p >= 0 for p in b.table("full", s))
    assert b.groups["win"].pool.n_free == 8 - 2 and b.groups["full"].pool.n_free == 8 - 5
    b.commit(s, 1)
    b.check()
    b.free_slot(s)
    assert b.groups["win"].pool.n_free == 8 and b.groups["full"].pool.n_free == 8


def test_random_walk_never_loses_or_doubles_anything():
    rng = random.Random(0)
    b = CacheBook([("full", None), ("win", 70)], n_pages=40, page_size=64, n_slots=6, max_seq_len=640)
    live = {}
    for _ in range(3000):
        r = rng.random()
        try:
            if r < 0.15 and b.n_free_slots:
                live[b.take_slot()] = 0
            elif r < 0.25 and live:
                s = rng.choice(list(live))
                b.free_slot(s)
                del live[s]
            elif live:
                s = rng.choice(list(live))
                n = rng.choice([1, 1, 1, 7, 64, 130])
                b.reserve(s, n)
                b.commit(s, n)
                live[s] += n
        except CacheError:
            pass
        b.check()
        for s, n in live.items():
            assert b.length(s) == n
    assert set(b.live_slots()) == set(live)


def test_a_refused_batch_takes_nothing():
    # two sequences at a page's end, one free page: the step that would need two pages is refused whole
    b = CacheBook([("full", None)], n_pages=3, page_size=64, n_slots=2, max_seq_len=256)
    s0, s1 = b.take_slot(), b.take_slot()
    b.reserve_batch([s0, s1], [64, 64])
    b.commit(s0, 64)
    b.commit(s1, 64)
    before = (b.table("full", s0), b.table("full", s1), b.groups["full"].pool.n_free)
    assert b.pages_short([s0, s1], [1, 1]) is not None
    with pytest.raises(CacheError, match="full"):
        b.reserve_batch([s0, s1], [1, 1])
    assert (b.table("full", s0), b.table("full", s1), b.groups["full"].pool.n_free) == before
    b.check()
    with pytest.raises(CacheError, match="limit"):
        b.reserve_batch([s0, s1], [1, 500])          # the second slot's fault: the first keeps its pages
    assert (b.table("full", s0), b.table("full", s1), b.groups["full"].pool.n_free) == before
    with pytest.raises(CacheError, match="twice"):
        b.reserve_batch([s0, s0], [1, 1])
    ch = b.reserve_batch([s0], [1])
    assert ch["full"] == [(s0, 1, 2)] and b.pages_short([s1], [1]) is not None
    b.check()


def test_a_window_gives_back_before_the_batch_takes():
    # the windowed pool is full, but the step itself releases the pages it then needs
    b = CacheBook([("win", 64)], n_pages=4, page_size=64, n_slots=2, max_seq_len=1024)
    s0, s1 = b.take_slot(), b.take_slot()
    b.reserve_batch([s0, s1], [128, 128])
    b.commit(s0, 128)
    b.commit(s1, 128)
    assert b.groups["win"].pool.n_free == 0 and b.pages_short([s0, s1], [1, 1]) is None
    ch = b.reserve_batch([s0, s1], [1, 1])["win"]
    assert sorted(c for c in ch if c[2] == -1) == [(s0, 0, -1), (s1, 0, -1)]
    assert sorted((c[0], c[1]) for c in ch if c[2] >= 0) == [(s0, 2), (s1, 2)]
    b.check()


def test_device_tables_follow_the_book_after_a_refusal():
    # the cache's mirror of the page tables (on the CPU here: no kernel runs) equals the book whatever was refused
    import torch
    from dlgo_b200.cache import KVCache
    from dlgo_b200.parts.base import CacheNeed
    kv = KVCache([CacheNeed("full", 1, 16)], [None], {}, max_tokens=3 * 64, max_seq_len=192, dtype=torch.float32,
                 device=torch.device("cpu"), n_slots=2)
    a, c = kv.take_slot(), kv.take_slot()
    kv.reserve([a, c], [64, 64])
    kv.commit([a, c], [64, 64])

    def mirrored():
        for s in (a, c):
            row = kv.page_tables["full"][s].tolist()
            held = kv.book.table("full", s)
            assert row[:len(held)] == held and all(p == -1 for p in row[len(held):]), (s, row, held)

    mirrored()
    with pytest.raises(CacheError, match="full"):
        kv.reserve([a, c], [1, 1])
    mirrored()
    assert kv.book.table("full", a) == [0] and kv.pages_short([a], [1]) is None
    kv.reserve([a], [1])
    kv.commit([a], [1])
    mirrored()
    assert kv.book.table("full", a)[1] >= 0
    kv.free_slot(a)
    kv.free_slot(c)
    kv.book.check()
    assert kv.page_tables["full"].eq(-1).all()
