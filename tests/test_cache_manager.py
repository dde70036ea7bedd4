"""The cache manager's accounting: no page lost, held twice or freed twice, under random orders of requests."""

from __future__ import annotations

import random

import pytest

from acvram_b200.cache import (CacheAccountingError, CacheManager, CachePlan, OutOfPages, PagedNeed, PagePool,
                               StateNeed)


def manager(num_pages=12, page=4, window=0, max_requests=4, layers=3, state=False):
    needs = [PagedNeed(2, 16, 0)] * layers
    if window:
        needs += [PagedNeed(2, 16, window)] * 2
    if state:
        needs += [StateNeed((3, 5))]
    return CacheManager(CachePlan(needs), page, num_pages, max_requests)


def test_pool_reuses_the_page_freed_last():
    pool = PagePool(4)
    a = pool.allocate(3)
    pool.release([a[1]])
    assert pool.allocate(1) == [a[1]]
    pool.check()


def test_double_free_and_foreign_free_are_caught():
    pool = PagePool(4)
    a = pool.allocate(2)
    pool.release(a)
    with pytest.raises(CacheAccountingError):
        pool.release([a[0]])
    with pytest.raises(CacheAccountingError):
        pool.release([99])


def test_allocation_is_all_or_nothing():
    m = manager(num_pages=3)
    m.admit("a")
    with pytest.raises(OutOfPages):
        m.grow("a", 13)
    assert m.free_pages() == [3]
    m.grow("a", 12)
    assert m.free_pages() == [0]
    m.check()


def test_groups_have_pages_of_their_own():
    m = manager(num_pages=10, window=6)
    assert len(m.paged_groups) == 2 and [g.num_slots for g in m.paged_groups] == [3, 2]
    m.admit("a")
    m.grow("a", 20)
    m.advance("a", 20)
    assert m.free_pages() == [5, 5]
    freed = m.trim("a")
    # window 6 at length 20: keys <= 14 are never read again -> pages 0..2 (positions 0..11) go back
    assert freed == 3 and m.free_pages() == [5, 8]
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and m.block_table("a", 1)[3] >= 0
    assert all(p >= 0 for p in m.block_table("a", 0))
    m.check()
    m.release("a")
    assert m.free_pages() == [10, 10]
    m.check()


def test_window_never_frees_a_page_a_later_query_reads():
    page, window = 4, 6
    m = manager(num_pages=64, page=page, window=window)
    m.admit("a")
    length = 0
    rng = random.Random(0)
    while length < 150:
        length += rng.choice([1, 1, 2, 5, 9])
        m.grow("a", length)
        m.advance("a", length)
        m.trim("a")
        table = m.block_table("a", 1)
        for j in range(max(0, length - window + 1), length):     # what the next query (position >= length) may read
            assert table[j // page] >= 0
        m.check()


def test_state_slots_follow_the_request():
    m = manager(state=True, max_requests=2)
    s1 = m.admit("a")
    s2 = m.admit("b")
    assert list(s1.values()) != list(s2.values())
    assert not m.can_admit()
    with pytest.raises(OutOfPages):
        m.admit("c")
    m.release("a")
    assert m.can_admit()
    s3 = m.admit("c")
    assert list(s3.values()) == list(s1.values()), "a freed slot is used again"
    with pytest.raises(CacheAccountingError):
        m.release("a")
    m.check()


def test_advance_beyond_pages_is_an_error():
    m = manager()
    m.admit("a")
    m.grow("a", 4)
    with pytest.raises(CacheAccountingError):
        m.advance("a", 5)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests(seed):
    """Requests come, grow by portions, and go in random order; the books always balance."""
    rng = random.Random(seed)
    m = manager(num_pages=24, page=4, window=rng.choice([0, 5, 9]), max_requests=5, state=seed % 2 == 0)
    live: dict[int, int] = {}
    next_id = 0
    held_before: dict[int, set] = {}
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.can_admit():
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.8 and live:
            r = rng.choice(list(live))
            n = live[r] + rng.choice([1, 1, 1, 3, 7, 16])
            if m.can_grow(r, n):
                m.grow(r, n)
                m.advance(r, n)
                m.trim(r)
                live[r] = n
            else:
                with pytest.raises(OutOfPages):
                    m.grow(r, n)
        elif live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        m.check()
        # no page in two tables
        for g in m.paged_groups:
            seen = set()
            for table in g.tables.values():
                for p in table:
                    if p >= 0:
                        assert p not in seen
                        seen.add(p)
    for r in list(live):
        m.release(r)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.paged_groups)
    assert all(g.num_free == g.max_requests for g in m.state_groups)
