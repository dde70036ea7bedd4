"""The scheduler's decisions, with a fake model: admission, portions under a token budget, decoding,
finishing and freeing, and what happens when pages run out."""

from __future__ import annotations

import random

import pytest

from acvram_b200.cache import CacheManager, CachePlan, PagedNeed
from acvram_b200.engine.scheduler import Request, Scheduler
from acvram_b200.sampling import SamplingParams


def make(num_pages=16, page=4, max_batch=4, budget=16, max_len=256):
    m = CacheManager(CachePlan([PagedNeed(1, 8, 0)] * 2), page, num_pages, max_batch)
    return m, Scheduler(m, max_batch, budget, max_len)


def req(i, n, max_tokens=4, **kw):
    return Request(f"r{i}", list(range(1, n + 1)), SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw), seed=i)


def run_step(m, s, token=7, eos=()):
    """Schedule, 'run' (advance the cache manager as the runner does) and commit."""
    plan = s.schedule()
    for e in plan.entries:
        m.advance(e.request.request_id, e.start + e.count)
    s.commit(plan, [token] * sum(e.samples for e in plan.entries), eos)
    m.check()
    return plan


def test_prompt_is_cut_into_portions_under_the_budget():
    m, s = make(budget=16, num_pages=32)
    s.add(req(0, 40))
    sizes = []
    while not s.idle:
        plan = run_step(m, s)
        sizes.append([(e.request.request_id, e.start, e.count, e.samples) for e in plan.entries])
    assert sizes[0] == [("r0", 0, 16, False)] and sizes[1] == [("r0", 16, 16, False)]
    assert sizes[2] == [("r0", 32, 8, True)]
    assert sizes[3] == [("r0", 40, 1, True)], "after the prompt, one token per step"
    assert len(sizes) == 3 + 3 and m.free_pages() == [32]


def test_decode_tokens_come_first_and_portions_share_the_rest():
    m, s = make(budget=10, num_pages=64)
    s.add(req(0, 6, max_tokens=10))
    run_step(m, s)                       # r0 whole prompt, first token
    s.add(req(1, 30))
    s.add(req(2, 5))
    plan = run_step(m, s)
    got = [(e.request.request_id, e.count, e.samples) for e in plan.entries]
    assert got == [("r0", 1, True), ("r1", 9, False)], "1 decode token, then 9 of the budget for the oldest prompt"
    plan = run_step(m, s)
    got = [(e.request.request_id, e.count) for e in plan.entries]
    assert got == [("r0", 1), ("r1", 9)]
    plan = run_step(m, s)
    plan = run_step(m, s)                # r1 has 3 left: r2 gets a portion in the same step
    got = [(e.request.request_id, e.count, e.samples) for e in plan.entries]
    assert got == [("r0", 1, True), ("r1", 3, True), ("r2", 5, True)]


def test_finish_reasons():
    m, s = make()
    s.add(req(0, 3, max_tokens=2, ignore_eos=True))
    s.add(req(1, 3, max_tokens=5))
    s.add(req(2, 3, max_tokens=5, ignore_eos=True))
    s.add(req(3, 3, max_tokens=5, stop_token_ids=[7]))
    reqs = list(s.waiting)
    run_step(m, s, token=9, eos=(9,))
    assert reqs[1].finish_reason == "stop" and reqs[1].output == [9]
    assert not reqs[2].finished
    run_step(m, s, token=7, eos=(9,))
    assert reqs[0].finish_reason == "length" and reqs[0].output == [9, 7]
    assert reqs[3].finish_reason == "stop"
    assert not reqs[2].finished
    while not s.idle:
        run_step(m, s, token=9, eos=(9,))
    assert reqs[2].finish_reason == "length" and len(reqs[2].output) == 5
    assert m.free_pages() == [16] and not m.live()


def test_max_tokens_zero_delivers_nothing():
    m, s = make()
    s.add(req(0, 3, max_tokens=0))
    r = s.waiting[0]
    run_step(m, s)
    assert r.finished and r.finish_reason == "length" and r.output == []


def test_request_that_can_never_fit_is_refused():
    m, s = make(num_pages=4, page=4)     # 16 tokens in all
    s.add(req(0, 20))
    s.add(req(1, 5))
    plan = s.schedule()
    assert [r.request_id for r in plan.refused] == ["r0"] and plan.refused[0].finish_reason == "refused"
    assert [e.request.request_id for e in plan.entries] == ["r1"]
    assert s.counters["refused"] == 1


def test_waiting_request_waits_for_pages():
    m, s = make(num_pages=6, page=4, budget=64)
    s.add(req(0, 15, max_tokens=3))
    s.add(req(1, 12, max_tokens=3))
    plan = run_step(m, s)
    assert [e.request.request_id for e in plan.entries] == ["r0"], "r1 needs 3 pages, 2 are free: it waits"
    assert len(s.waiting) == 1
    while s.running:
        run_step(m, s)
    plan = run_step(m, s)
    assert [e.request.request_id for e in plan.entries] == ["r1"]


def test_pages_run_out_while_decoding_preempts_the_latest():
    """Two requests fill the pool; when the older one needs a page the later one is preempted,
    requeued at the head, and recomputed with its tokens so far."""
    m, s = make(num_pages=4, page=4, budget=64)
    s.add(req(0, 7, max_tokens=8))
    s.add(req(1, 6, max_tokens=8))
    r0, r1 = list(s.waiting)
    run_step(m, s)                         # both prompts: 2 + 2 pages
    assert m.free_pages() == [0]
    plan = run_step(m, s)                  # r0: 8 tokens, fits; r1: 7 tokens, fits
    assert not plan.preempted
    plan = run_step(m, s)                  # r0 needs a third page -> r1 (admitted last) gives way
    assert [r.request_id for r in plan.preempted] == ["r1"]
    assert [e.request.request_id for e in plan.entries] == ["r0"]
    assert r1.computed == 0 and r1.preemptions == 1 and s.waiting[0] is r1 and len(r1.output) == 2
    assert s.counters["preempted"] == 1
    while not s.idle:
        run_step(m, s)
    assert len(r0.output) == 8 and len(r1.output) == 8, "the preempted request still gets all its tokens"
    assert m.free_pages() == [4]


def test_request_alone_that_cannot_grow_is_cut_and_delivered():
    m, s = make(num_pages=2, page=4, budget=64)
    s.add(req(0, 6, max_tokens=20))
    r = s.waiting[0]
    plans = []
    while not s.idle:
        plans.append(run_step(m, s))
    assert r.finish_reason == "length" and len(r.prompt) + len(r.output) == 9
    assert plans[-1].truncated == [r] and s.counters["truncated"] == 1
    assert m.free_pages() == [2]


def test_abort_frees_pages():
    m, s = make(budget=32)
    s.add(req(0, 9))
    s.add(req(1, 9))
    run_step(m, s)
    s.abort("r0")
    m.check()
    assert len(s.running) == 1 and m.free_pages() == [16 - 3]
    s.abort("r1")
    assert s.idle and m.free_pages() == [16]


def test_too_long_prompt_is_an_error():
    m, s = make(max_len=10)
    with pytest.raises(ValueError):
        s.add(req(0, 10))


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_ends_with_every_page_free(seed):
    rng = random.Random(seed)
    m, s = make(num_pages=rng.choice([6, 9, 20]), page=4, max_batch=rng.choice([2, 4]), budget=rng.choice([3, 8, 32]))
    reqs = [req(i, rng.randint(1, 18), max_tokens=rng.randint(1, 12)) for i in range(12)]
    pending = list(reqs)
    steps = 0
    while pending or not s.idle:
        if pending and rng.random() < 0.5:
            s.add(pending.pop(0))
        plan = run_step(m, s, token=rng.randint(1, 50))
        assert plan.num_tokens <= s.token_budget
        assert len(s.running) <= s.max_batch_size
        steps += 1
        assert steps < 3000
    for r in reqs:
        assert r.finished
        if r.finish_reason == "length" and len(r.prompt) + len(r.output) < 24:
            assert len(r.output) == r.params.max_tokens or m.paged_groups[0].pool.num_pages * 4 <= len(r.prompt) + len(r.output) + 4
    assert m.free_pages() == [m.paged_groups[0].pool.num_pages] and not m.live()


# ----------------------------------------------------------------------------- one step ahead
def _decode_state(n_req=3, prompt=5, max_tokens=6, **kw):
    m, s = make(num_pages=32, page=4, max_batch=4, budget=64, **kw)
    rs = [req(i, prompt, max_tokens=max_tokens) for i in range(n_req)]
    for r in rs:
        s.add(r)
    run_step(m, s)                      # the prompts, first tokens
    return m, s, rs


def test_step_planned_ahead_of_the_tokens_before_it():
    m, s, rs = _decode_state()
    prev = s.schedule()
    assert s.schedule_ahead_possible(prev)
    ahead = s.schedule_ahead(prev)
    assert [(e.request, e.start, e.count, e.samples) for e in ahead.entries] == \
        [(e.request, e.start + 1, 1, True) for e in prev.entries]
    s.commit(prev, [7] * 3)
    s.commit(ahead, [8] * 3)
    assert all(r.output[-2:] == [7, 8] and r.computed == len(r.tokens) - 1 for r in rs)
    m.check()


def test_ahead_leaves_out_requests_at_their_length_and_ignores_stopped_ones():
    m, s, rs = _decode_state(max_tokens=3)
    rs[1].params = SamplingParams(max_tokens=2)            # its next token is its last
    prev = s.schedule()
    ahead = s.schedule_ahead(prev)
    assert [e.request for e in ahead.entries] == [rs[0], rs[2]]
    # rs[0] stops on the token of prev (end of sequence): the step planned ahead still holds it, its token is dropped
    s.commit(prev, [99, 7, 7], eos_token_ids=(99,))
    assert rs[0].finished and rs[0].finish_reason == "stop" and rs[1].finished and rs[1].finish_reason == "length"
    touched = s.commit(ahead, [5, 6])
    assert touched == [rs[2]] and rs[2].output[-1] == 6 and rs[0].output[-1] == 99
    m.check()
    assert s.running == [] or s.running == [rs[2]] or rs[2].finished


def test_no_step_ahead_while_someone_waits_or_a_prompt_runs_or_pages_lack():
    m, s, rs = _decode_state()
    s.add(req(9, 4))
    prev = s.schedule()                                     # admits the newcomer: a prompt portion is in the plan
    assert not s.schedule_ahead_possible(prev) and s.schedule_ahead(prev) is None
    run = s.commit(prev, [7] * len([e for e in prev.entries if e.samples]))
    # pages: a pool that holds exactly what is used now lets nobody grow across a page's edge
    m2, s2 = make(num_pages=4, page=4, max_batch=2, budget=64)
    a, b = req(0, 7, max_tokens=8), req(1, 7, max_tokens=8)
    s2.add(a); s2.add(b)
    run_step(m2, s2)                                        # 8 tokens each: two full pages each, pool empty
    prev = s2.schedule()                                    # may preempt to go on; whatever it does, ahead must not steal
    if prev.entries and not prev.preempted:
        assert s2.schedule_ahead(prev) is None
    m2.check()


def test_ahead_counts_the_pages_of_all_requests_together():
    """Two requests that each need a new page for the step ahead, one free page: no step ahead (and nothing taken)."""
    m, s = make(num_pages=5, page=4, max_batch=2, budget=64)
    a, b = req(0, 3, max_tokens=8), req(1, 3, max_tokens=8)
    s.add(a); s.add(b)
    run_step(m, s)                  # 3 tokens each in the cache, one page each; both now bring their 4th token
    prev = s.schedule()             # positions 3: still the first page
    free = m.free_pages()
    assert free == [3]
    m.paged_groups[0].pool.allocate(2)          # somebody else's pages: one page left for two requests that both need one
    assert s.schedule_ahead(prev) is None and m.free_pages() == [1]


# --------------------------------------------------------------------------- prefix reuse
def make_reuse(num_pages=16, page=4, max_batch=4, budget=16, max_len=256):
    m = CacheManager(CachePlan([PagedNeed(1, 8, 0)] * 2), page, num_pages, max_batch, enable_prefix_cache=True)
    return m, Scheduler(m, max_batch, budget, max_len)


def test_a_prompt_seen_before_starts_behind_its_known_pages():
    m, s = make_reuse(budget=64, num_pages=32)
    s.add(req(0, 22, max_tokens=3))
    while not s.idle:
        run_step(m, s)
    # r0 held 22 prompt tokens and fed two of its three tokens: 24 tokens in six full pages
    assert m.paged_groups[0].pool.num_kept == 6 and m.free_pages() == [32]
    r1 = req(1, 22, max_tokens=2)
    s.add(r1)
    plan = run_step(m, s)
    assert [(e.start, e.count, e.samples) for e in plan.entries] == [(20, 2, True)], "five pages taken over, two tokens run"
    assert r1.reused == 20 and s.counters["reused_tokens"] == 20
    r2 = Request("r2", list(range(1, 11)) + [90, 91, 92], SamplingParams(temperature=0.0, max_tokens=2))
    s.add(r2)
    plan = run_step(m, s)
    assert [(e.request.request_id, e.start, e.count) for e in plan.entries] == [("r1", 22, 1), ("r2", 8, 5)]
    while not s.idle:
        run_step(m, s)
    assert m.free_pages() == [32]


def test_a_preempted_request_takes_its_own_pages_back():
    m, s = make_reuse(num_pages=6, page=4, budget=32)
    a, b = req(0, 7, max_tokens=12), req(1, 7, max_tokens=12)
    s.add(a)
    s.add(b)
    run_step(m, s)                      # both prompts: 2 pages each
    plan = None
    for _ in range(8):
        plan = run_step(m, s)
        if plan.preempted:
            break
    assert plan is not None and plan.preempted == [b]
    done = len(b.tokens)
    while not a.finished:
        run_step(m, s)
    while b.admitted_at < 0:
        run_step(m, s)
    assert b.reused >= (done - 1) // 4 * 4 - 4 and b.reused > 0, "its published pages were still there"
    while not s.idle:
        run_step(m, s)
    assert len(a.output) == 12 and len(b.output) == 12 and m.free_pages() == [6]


def test_random_traffic_with_shared_beginnings_keeps_the_books():
    """Random requests with shared beginnings, stops, aborts and a pool that preempts.  A shadow of what each page
    holds (written as the runner would write it) shows that a step never writes a page that two requests hold, that
    every position a step reads holds the tokens of the request that reads it, and the budget is kept."""
    reused = preempted = 0
    for seed in range(6):
        rng = random.Random(seed)
        page = 4
        m, s = make_reuse(num_pages=rng.choice([12, 20, 40]), page=page, max_batch=4, budget=rng.choice([5, 12, 30]), max_len=64)
        stems = [[rng.randrange(1, 40) for _ in range(20)] for _ in range(2)]
        shadow: dict[int, list] = {}                    # page -> the token whose keys each of its rows holds
        reqs = []
        for i in range(120):
            if rng.random() < 0.4 and len(s.waiting) < 3:
                prompt = rng.choice(stems)[:rng.randrange(1, 20)] + [rng.randrange(40, 60) for _ in range(rng.randrange(0, 4))]
                r = Request(f"q{seed}-{i}", prompt, SamplingParams(temperature=0.0, max_tokens=rng.randrange(1, 9),
                                                                   stop_token_ids=[7] if rng.random() < 0.3 else []))
                reqs.append(r)
                s.add(r)
            if rng.random() < 0.05 and s.running:
                s.abort(rng.choice(s.running).request_id)
            plan = s.schedule()
            assert plan.num_tokens <= s.token_budget and len(s.running) <= 4
            for e in plan.entries:
                r, table = e.request, m.block_table(e.request.request_id, 0)
                tokens = r.tokens
                for pos in range(e.start):              # what the step reads was written with this request's tokens
                    assert shadow[table[pos // page]][pos % page] == tokens[pos], (seed, i, r.request_id, pos)
                for pos in range(e.start, e.start + e.count):
                    p = table[pos // page]
                    assert m.paged_groups[0].pool.holders(p) == 1, "a page that two requests hold is written"
                    shadow.setdefault(p, [None] * page)[pos % page] = tokens[pos]
                m.advance(r.request_id, e.start + e.count)
            s.commit(plan, [rng.randrange(1, 40) for e in plan.entries if e.samples])
            m.check()
        steps = 0
        while not s.idle:
            plan = s.schedule()
            for e in plan.entries:
                table, tokens = m.block_table(e.request.request_id, 0), e.request.tokens
                for pos in range(e.start):
                    assert shadow[table[pos // page]][pos % page] == tokens[pos]
                for pos in range(e.start, e.start + e.count):
                    assert m.paged_groups[0].pool.holders(table[pos // page]) == 1
                    shadow.setdefault(table[pos // page], [None] * page)[pos % page] = tokens[pos]
                m.advance(e.request.request_id, e.start + e.count)
            s.commit(plan, [rng.randrange(1, 40) for e in plan.entries if e.samples])
            m.check()
            steps += 1
            assert steps < 2000
        assert all(r.finished for r in reqs) and m.free_pages() == [m.paged_groups[0].pool.num_pages]
        assert all(len(r.output) == r.params.max_tokens for r in reqs if r.finish_reason == "length")
        reused += s.counters["reused_tokens"]
        preempted += s.counters["preempted"]
    assert reused > 100 and preempted > 0


def test_full_pages_are_known_while_their_request_still_runs():
    m, s = make_reuse(budget=12, num_pages=32)
    a = req(0, 21, max_tokens=8)
    s.add(a)
    run_step(m, s)                                  # 12 of a's 21 prompt tokens: three pages, known at once
    b = req(1, 21, max_tokens=2)
    s.add(b)
    plan = run_step(m, s)                           # a's last 9 tokens; b takes a's three pages and runs 3 tokens
    assert [(e.request.request_id, e.start, e.count) for e in plan.entries] == [("r0", 12, 9), ("r1", 12, 3)]
    assert b.reused == 12 and m.block_table("r1", 0)[:3] == m.block_table("r0", 0)[:3]
    assert m.paged_groups[0].pool.holders(m.block_table("r0", 0)[0]) == 2
    while not s.idle:
        run_step(m, s)
    assert len(a.output) == 8 and len(b.output) == 2 and m.free_pages() == [32]


def test_a_failed_step_gives_its_pages_back_unpublished_and_leaves_the_others():
    """Scheduler.fail: the named requests end with "error", their pages are free again and not known to later
    requests; a running request that is not named and a waiting one go on (acvram/engine/runner.py:1329-1338)."""
    m = CacheManager(CachePlan([PagedNeed(1, 8, 0)] * 2), 4, 16, 4, enable_prefix_cache=True)
    s = Scheduler(m, 2, 8, 256)
    a, b, c = req(0, 11), Request("rb", list(range(50, 56)), SamplingParams(temperature=0.0, max_tokens=3), 1), req(2, 5)
    for r in (a, b, c):
        s.add(r)
    run_step(m, s)                                   # a's first 8 tokens: two full pages, published as they fill
    plan = s.schedule()                              # a's last 3 tokens and b's first 5
    assert {e.request.request_id for e in plan.entries} == {"r0", "rb"}
    free_before = m.free_pages()[0]
    ended = s.fail([e.request for e in plan.entries if e.request is a])
    assert ended == [a] and a.finished and a.finish_reason == "error" and a not in s.running
    assert b in s.running and c in s.waiting and s.counters["failed"] == 1
    m.check()
    assert m.free_pages()[0] == free_before + 3      # all three pages of a are back
    keys = m.page_keys(a.tokens)
    pool = m.paged_groups[0].pool
    assert pool.lookup(keys[0]) is not None and pool.lookup(keys[1]) is not None     # from the good step
    assert len(keys) == 2                             # the third page never filled: nothing of the failed step is known
    assert s.fail([a]) == []                          # ending it twice does nothing
    # b and c run to their ends
    for e in plan.entries:
        if e.request is b:
            m.advance("rb", e.start + e.count)
    s.commit(type(plan)([e for e in plan.entries if e.request is b]), [7], ())
    for _ in range(20):
        if s.idle:
            break
        run_step(m, s)
    assert s.idle and b.finish_reason == "length" and c.finish_reason == "length"
    m.check()
