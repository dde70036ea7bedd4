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


# --------------------------------------------------------------------------- prefix reuse
def reuse_manager(num_pages=12, page=4, max_requests=4, layers=2):
    return CacheManager(CachePlan([PagedNeed(2, 16, 0)] * layers), page, num_pages, max_requests, enable_prefix_cache=True)


def run_request(m, name, tokens, upto=None):
    """Admit ``name`` with ``tokens``, hold positions [0, upto); returns how many tokens it took over."""
    keys = m.page_keys(tokens)
    m.admit(name, keys, len(tokens))
    reused = m.lengths[name]
    upto = len(tokens) if upto is None else upto
    m.grow(name, upto)
    m.advance(name, upto)
    return reused


def test_a_finished_request_leaves_its_full_pages_to_the_next_with_the_same_beginning():
    m = reuse_manager()
    a = list(range(100, 111))                       # 11 tokens: two full pages and three tokens
    assert run_request(m, "a", a) == 0
    table_a = list(m.block_table("a", 0))
    m.release("a", m.page_keys(a))
    assert m.free_pages() == [12] and m.paged_groups[0].pool.num_kept == 2
    m.check()
    b = a[:9] + [7, 8, 9]                           # the same two pages, then something else
    assert run_request(m, "b", b) == 8
    assert m.block_table("b", 0)[:2] == table_a[:2] and m.block_table("b", 0)[2] not in table_a[:2]
    assert m.reused_tokens == 8
    m.check()
    c = a[:4] + [1, 2, 3, 4, 5]                     # only the first page is the same
    assert run_request(m, "c", c) == 4
    assert m.block_table("c", 0)[0] == table_a[0] and m.paged_groups[0].pool.holders(table_a[0]) == 2
    m.check()
    m.release("b", m.page_keys(b))
    assert m.paged_groups[0].pool.holders(table_a[0]) == 1, "c still holds the first page"
    m.release("c", m.page_keys(c))
    m.check()
    assert m.free_pages() == [12]


def test_the_last_token_of_a_known_prompt_is_still_computed():
    m = reuse_manager()
    a = list(range(8))                              # exactly two pages
    run_request(m, "a", a)
    m.release("a", m.page_keys(a))
    assert run_request(m, "b", list(a)) == 4, "the second page holds the last token: it is computed again"
    assert run_request(m, "c", a + [99]) == 8
    m.check()


def test_kept_pages_give_way_when_room_is_needed_the_deepest_first():
    m = reuse_manager(num_pages=4)
    a = list(range(12))
    run_request(m, "a", a)
    m.release("a", m.page_keys(a))
    pool = m.paged_groups[0].pool
    assert pool.num_kept == 3 and m.free_pages() == [4]
    m.admit("x")
    m.grow("x", 8)                                  # the free page, then the room of a's third page
    m.advance("x", 8)
    assert pool.num_kept == 2
    keys = m.page_keys(a + [1])
    assert m.reusable(keys, 13)[0] == 8, "the first two pages of a are still known"
    m.grow("x", 16)
    m.advance("x", 16)
    assert pool.num_kept == 0 and m.reusable(keys, 13)[0] == 0
    with pytest.raises(OutOfPages):
        m.grow("x", 17)
    m.check()
    m.release("x")
    assert m.free_pages() == [4] and pool.num_kept == 0, "pages released without tokens are not published"
    m.check()


def test_admission_counts_the_kept_pages_it_takes_over():
    m = reuse_manager(num_pages=4)
    a = list(range(12))
    run_request(m, "a", a)
    m.release("a", m.page_keys(a))                  # 3 kept, 1 free
    keys = m.page_keys(a + [50, 51, 52, 53, 54])
    # taking the three kept pages over leaves one page: room for up to 4 new tokens
    assert m.can_admit_with(keys, 17, 4) and not m.can_admit_with(keys, 17, 5)
    other = m.page_keys(list(range(200, 217)))
    assert m.can_admit_with(other, 17, 16) and not m.can_admit_with(other, 17, 17)


def test_reuse_is_off_for_windows_and_states_and_by_default():
    assert not manager().prefix_reuse
    plan = CachePlan([PagedNeed(2, 16, 0), PagedNeed(2, 16, 6)])
    assert not CacheManager(plan, 4, 8, 2, enable_prefix_cache=True).prefix_reuse
    plan = CachePlan([PagedNeed(2, 16, 0), StateNeed((3,))])
    assert not CacheManager(plan, 4, 8, 2, enable_prefix_cache=True).prefix_reuse
    m = manager()
    a = list(range(9))
    m.admit("a", m.page_keys(a), 9)
    m.grow("a", 9); m.advance("a", 9)
    m.release("a", m.page_keys(a))
    assert m.paged_groups[0].pool.num_kept == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_shared_beginnings(seed):
    """Requests whose tokens begin alike come and go at random; a page taken over always holds the
    tokens of the request that takes it (checked against a shadow of what was written where)."""
    rng = random.Random(seed)
    page = 4
    m = reuse_manager(num_pages=14, page=page, max_requests=4)
    stems = [[rng.randrange(50) for _ in range(24)] for _ in range(3)]
    written: dict[int, tuple] = {}                  # page -> the tokens from position 0 to the page's end
    live: dict[int, tuple[list, int]] = {}
    next_id = 0
    for _ in range(500):
        action = rng.random()
        if action < 0.3 and m.can_admit():
            stem = rng.choice(stems)
            tokens = stem[:rng.randrange(1, 24)] + [rng.randrange(50, 99) for _ in range(rng.randrange(0, 9))]
            keys = m.page_keys(tokens)
            if m.can_admit_with(keys, len(tokens), 1):
                m.admit(next_id, keys, len(tokens))
                have = m.lengths[next_id]
                assert have % page == 0 and have < len(tokens)
                for i, p in enumerate(m.block_table(next_id, 0)):
                    assert written[p] == tuple(tokens[:(i + 1) * page]), "a page taken over holds other tokens"
                live[next_id] = (tokens, have)
                next_id += 1
        elif action < 0.8 and live:
            r = rng.choice(list(live))
            tokens, have = live[r]
            n = min(len(tokens), have + rng.choice([1, 2, 5, 9]))
            if n > have and m.can_grow(r, n):
                m.grow(r, n)
                m.advance(r, n)
                table = m.block_table(r, 0)
                for i in range(have // page, (n - 1) // page + 1):
                    assert m.paged_groups[0].pool.holders(table[i]) == 1, "a shared page is written"
                    written[table[i]] = tuple(tokens[:min(n, (i + 1) * page)])
                live[r] = (tokens, n)
                if rng.random() < 0.5:              # full pages become known while the request still runs
                    m.publish(r, m.page_keys(tokens), n)
        elif live:
            r = rng.choice(list(live))
            tokens, have = live.pop(r)
            m.release(r, m.page_keys(tokens) if rng.random() < 0.8 else ())
        m.check()
    for r, (tokens, _) in live.items():
        m.release(r, m.page_keys(tokens))
    m.check()
    assert m.free_pages() == [14] and m.reused_tokens > 0


def test_changed_block_table_entries_go_out_once_each():
    """The device's copy of the block tables gets (row, column, page) triples; an entry that changed twice between
    two steps (a row given back and taken again) goes out once, with its last value."""
    m = CacheManager(CachePlan([PagedNeed(1, 8, 0)]), 4, 8, 2)
    m.admit("a")
    m.grow("a", 6)
    row_a = m.rows["a"]
    first = m.take_updates()[0]
    assert sorted(first) == [(row_a, 0, m.block_table("a", 0)[0]), (row_a, 1, m.block_table("a", 0)[1])]
    assert m.take_updates() == [[]]
    m.admit("b")
    m.grow("b", 3)
    m.release("b")                      # given back before any step ran
    m.admit("c")                        # takes the same row
    m.grow("c", 9)
    assert m.rows["c"] != row_a
    got = m.take_updates()[0]
    assert len(got) == len({(r, c) for r, c, _ in got}) == 3
    assert sorted(got) == [(m.rows["c"], i, p) for i, p in enumerate(m.block_table("c", 0))]
    m.resync()
    again = m.take_updates()[0]
    assert sorted(again) == sorted([(row_a, i, p) for i, p in enumerate(m.block_table("a", 0))] +
                                   [(m.rows["c"], i, p) for i, p in enumerate(m.block_table("c", 0))])
    m.check()
