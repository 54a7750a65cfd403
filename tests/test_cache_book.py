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
