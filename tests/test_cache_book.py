"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; windows give pages back."""

import random

import numpy as np
import pytest

from sleuth_b200.cache.book import CacheBook, CacheFull, CacheMisuse, PagePool, pages_for


def invariants(book: CacheBook):
    live = book.live_slots()
    assert len(live) + book.free_slots == book.max_slots
    for g in book.groups:
        held = []
        for s in range(book.max_slots):
            row = g.table[s]
            pages = row[row >= 0].tolist()
            if s not in live:
                assert not pages, "a free slot still holds pages"
            held += pages
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) + g.pool.free == g.pool.n_pages, "a page was lost"
        assert sorted(held + g.pool._free) == list(range(g.pool.n_pages))


def test_pool_take_give():
    p = PagePool(4)
    a = p.take(3)
    assert len(set(a)) == 3 and p.free == 1
    with pytest.raises(CacheFull):
        p.take(2)
    p.give(a[:1])
    with pytest.raises(CacheMisuse):
        p.give(a[:1])
    assert p.take(1) == a[:1]          # the lowest free page is used again first


def test_pool_hands_out_the_lowest_pages_so_that_held_pages_stay_together():
    p = PagePool(64)
    first, second, third = p.take(10), p.take(10), p.take(10)
    assert first == list(range(10)) and second == list(range(10, 20)) and third == list(range(20, 30))
    p.give(second)
    p.give(first[3:7])
    # what comes back is used before untouched pages, in ascending order whatever the order of the returns
    assert p.take(6) == [3, 4, 5, 6, 10, 11]
    assert p.take(10) == [12, 13, 14, 15, 16, 17, 18, 19, 30, 31]
    assert p.free == 64 - 32


def test_slots_are_reused_and_lengths_start_at_zero():
    book = CacheBook([0], n_pages=8, max_slots=3, stride=4)
    s = book.open(3)
    assert sorted(s) == [0, 1, 2]
    with pytest.raises(CacheFull):
        book.open(1)
    book.grow(s, [70, 1, 64])
    book.commit(s, [70, 1, 64])
    assert book.pages_in_use() == [2 + 1 + 1] and book.lengths[s[0]] == 70
    book.close([s[1]])
    with pytest.raises(CacheMisuse):
        book.close([s[1]])
    again = book.open(1)
    assert again == [s[1]] and book.lengths[again[0]] == 0 and (book.groups[0].table[again[0]] == -1).all()
    invariants(book)


def test_growth_is_all_or_nothing():
    book = CacheBook([0], n_pages=3, max_slots=2, stride=4)
    a, b = book.open(2)
    book.grow([a], [64])
    book.commit([a], [64])
    with pytest.raises(CacheFull):
        book.grow([a, b], [128, 129])        # needs 1 + 3 pages, 2 are free
    assert book.pages_in_use() == [1]
    invariants(book)
    with pytest.raises(CacheFull):
        book.grow([a], [4 * 64 + 1])         # longer than the longest sequence allowed
    with pytest.raises(CacheMisuse):
        book.grow([a], [10])                 # shrinking


def test_window_group_gives_pages_back_and_keeps_positions():
    book = CacheBook([0, 100], n_pages=40, max_slots=2, stride=32)
    (s,) = book.open(1)
    n = 0
    for step in [500] + [1] * 400:
        n += step
        book.grow([s], [n])
        book.commit([s], [n])
        full, win = book.groups
        assert (full.table[s] >= 0).sum() == pages_for(n)
        first = max(0, n - 100 + 1) // 64
        held = np.nonzero(win.table[s] >= 0)[0]
        assert held.min() == first and held.max() == pages_for(n) - 1      # entry i still means positions 64i..64i+63
        assert len(held) <= pages_for(100) + 1
        invariants(book)
    book.close([s])
    assert book.pages_in_use() == [0, 0]


def test_tables_for_returns_rows_in_batch_order():
    book = CacheBook([0], n_pages=16, max_slots=4, stride=4)
    s = book.open(3)
    book.grow(s, [65, 1, 200])
    t = book.tables_for([s[2], s[0]])[0]
    assert t.shape == (2, 4) and (t[0] >= 0).sum() == 4 and (t[1] >= 0).sum() == 2


def test_random_schedule_keeps_the_books():
    rng = random.Random(3)
    book = CacheBook([0, 70], n_pages=64, max_slots=6, stride=16)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.2 and book.free_slots:
            for s in book.open(rng.randint(1, book.free_slots)):
                live[s] = 0
        elif op < 0.8 and live:
            batch = rng.sample(sorted(live), rng.randint(1, len(live)))
            new = [min(live[s] + rng.choice([1, 1, 1, 7, 64, 130]), 16 * 64) for s in batch]
            try:
                book.grow(batch, new)
            except CacheFull:
                invariants(book)
                continue
            book.commit(batch, new)
            for s, n in zip(batch, new):
                live[s] = n
        elif live:
            gone = rng.sample(sorted(live), rng.randint(1, len(live)))
            book.close(gone)
            for s in gone:
                del live[s]
        invariants(book)
        for s, n in live.items():
            assert book.lengths[s] == n
    book.close(sorted(live))
    assert book.pages_in_use() == [0, 0] and book.free_slots == 6
