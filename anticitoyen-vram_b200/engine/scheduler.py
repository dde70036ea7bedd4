"""The scheduler: which tokens of which requests the next step runs.

Queues and life of a request follow the reference (waiting FIFO, running list,
single-threaded; acvram/engine/runner.py:819-820, 1346-1459, 1945-2074), with two
differences that the mixed step function allows:

* one token budget per step over the whole batch: every running request that has
  only its last token left gets that one token first, the rest of the budget is
  cut into prompt portions, first come first served, so portions change size from
  step to step (the reference's ``ACVRAM_BUDGET_JETONS`` is per request and runs
  each portion alone, acvram/engine/runner.py:1992-2046);
* when pages run out while requests decode, the request admitted last is
  *preempted*: its pages go back, it returns to the head of the waiting queue and
  its tokens so far are recomputed as a prompt later.  The reference truncates the
  request instead (finish reason "length", acvram/engine/runner.py:1727-1753); here
  that happens only to a request that is alone and still cannot grow.  A request
  that could not be held even by an empty pool is refused at once (the reference's
  named refusal, acvram/engine/runner.py:1356-1369).  Nothing is silent: every
  such decision is in the step's plan and in the counters.

The scheduler owns no device memory: it reserves pages in the cache manager and
hands the runner a list of (request, tokens, want).
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Hashable, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass(eq=False)        # a request is itself: membership in the queues is by identity, not by comparing token lists
class Request:
    request_id: Hashable
    prompt: list[int]
    params: SamplingParams
    seed: int = 0
    output: list[int] = field(default_factory=list)
    computed: int = 0            # tokens of prompt+output whose keys and values are in the cache
    admitted_at: int = -1        # admission order (larger = later); -1 while waiting
    finished: bool = False
    finish_reason: str | None = None
    preemptions: int = 0
    logprob_sum: float = 0.0
    reused: int = 0              # tokens taken over from published pages at the last admission
    page_keys: list = field(default_factory=list, repr=False)   # keys of the full pages of ``tokens``, as far as made
    published: int = 0           # pages of this admission that are already known to later requests
    text: str = ""               # the output's text so far (when the engine has a tokenizer)
    text_tokens: int = 0         # output tokens that ``text`` covers

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        return len(self.prompt) + len(self.output) - self.computed

    def token_slice(self, start: int, count: int) -> list[int]:
        """tokens[start : start + count] without putting prompt and output together first."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]


@dataclass
class PlannedEntry:
    request: Request
    start: int
    count: int
    samples: bool        # the portion reaches the request's last token: its logits are wanted


@dataclass
class StepPlan:
    entries: list[PlannedEntry] = field(default_factory=list)
    preempted: list[Request] = field(default_factory=list)
    refused: list[Request] = field(default_factory=list)
    truncated: list[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, manager: CacheManager, max_batch_size: int, token_budget: int, max_model_len: int) -> None:
        if token_budget < 1 or max_batch_size < 1:
            raise ValueError("token_budget and max_batch_size must be >= 1")
        self.manager = manager
        self.max_batch_size = max_batch_size
        self.token_budget = token_budget
        self.max_model_len = max_model_len
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._order = itertools.count()
        self.counters = {"preempted": 0, "refused": 0, "truncated": 0, "admitted": 0, "reused_tokens": 0, "failed": 0}

    # ------------------------------------------------------------------ queue
    def add(self, request: Request) -> None:
        if len(request.prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        if len(request.prompt) >= self.max_model_len:
            # the reference raises for the same case (acvram/engine/runner.py:1305-1308)
            raise ValueError(f"prompt of {len(request.prompt)} tokens does not fit max_model_len {self.max_model_len}")
        self.waiting.append(request)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def abort(self, request_id: Hashable) -> Request | None:
        for r in list(self.running):
            if r.request_id == request_id:
                self._finish(r, "abort")
                return r
        for r in list(self.waiting):
            if r.request_id == request_id:
                self.waiting.remove(r)
                r.finished, r.finish_reason = True, "abort"
                return r
        return None

    # ------------------------------------------------------------------ one step's plan
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        m = self.manager
        budget = self.token_budget

        # 1. single tokens of the requests that have only their last token left
        for r in sorted(self.running, key=lambda r: r.admitted_at):
            if r not in self.running or r.remaining != 1 or r.computed == 0:
                continue
            if budget == 0:
                break
            while not m.can_grow(r.request_id, r.computed + 1):
                victim = max(self.running, key=lambda q: q.admitted_at)
                if victim is r and len(self.running) == 1:
                    self._finish(r, "length")        # alone and still no page: delivered, counted
                    plan.truncated.append(r)
                    self.counters["truncated"] += 1
                    break
                self._preempt(victim, plan)
                if victim is r:
                    break
            if r.finished or r not in self.running:
                continue
            m.grow(r.request_id, r.computed + 1)
            plan.entries.append(PlannedEntry(r, r.computed, 1, True))
            budget -= 1

        # 2. portions of prompts already begun, oldest first
        for r in sorted(self.running, key=lambda r: r.admitted_at):
            if budget == 0:
                break
            if r.remaining == 1 and r.computed > 0 or any(e.request is r for e in plan.entries):
                continue
            budget -= self._plan_portion(r, budget, plan)

        # 3. new requests, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_size and m.can_admit():
            r = self.waiting[0]
            if not m.fits_empty_pool(r.num_tokens + 1):
                self.waiting.popleft()
                r.finished, r.finish_reason = True, "refused"
                plan.refused.append(r)
                self.counters["refused"] += 1
                continue
            keys = self._keys(r)
            n_tokens = r.num_tokens
            reuse, _ = m.reusable(keys, n_tokens)
            first = min(n_tokens - reuse, budget)
            if not m.can_admit_with(keys, n_tokens, first):
                break                                # stays waiting until pages come back
            self.waiting.popleft()
            m.admit(r.request_id, keys, n_tokens)
            r.computed = r.reused = m.lengths[r.request_id]     # published pages of the same beginning, taken over
            r.published = r.reused // m.page_size
            self.counters["reused_tokens"] += r.reused
            r.admitted_at = next(self._order)
            self.running.append(r)
            self.counters["admitted"] += 1
            budget -= self._plan_portion(r, budget, plan)

        # 4. nothing could run although requests are live: two unfinished prompts hold the pool
        #    between them; the later one gives way
        if not plan.entries and len(self.running) > 1:
            self._preempt(max(self.running, key=lambda q: q.admitted_at), plan)
            return self.schedule_after_preemption(plan)
        if not plan.entries and len(self.running) == 1 and not plan.truncated:
            r = self.running[0]
            self._finish(r, "length")
            plan.truncated.append(r)
            self.counters["truncated"] += 1
        return plan

    def schedule_ahead_possible(self, prev: StepPlan) -> bool:
        """Whether ``prev`` is of the kind after which a step can be planned ahead (see ``schedule_ahead``)."""
        return (not self.waiting and bool(prev.entries) and len(prev.entries) == len(self.running)
                and not (prev.preempted or prev.refused or prev.truncated)
                and all(e.count == 1 and e.samples for e in prev.entries))

    def schedule_ahead(self, prev: StepPlan) -> StepPlan | None:
        """The step after ``prev``, planned before ``prev``'s tokens are known, or None when that cannot be done.

        It can when ``prev`` is single tokens of every running request and nobody waits: each request then
        brings its next token, whatever it is (the engine feeds it on the device).  Requests that ``prev``
        brings to their length limit are left out; one that stops on a token of its own (end of sequence, a
        stop token) is found out only when ``prev`` is committed, and its entry here is then ignored
        (``commit`` skips finished requests).  Nothing is preempted here: if a page is missing the caller
        falls back to ``schedule``."""
        if self.waiting or not prev.entries or prev.preempted or prev.refused or prev.truncated:
            return None
        if len(prev.entries) != len(self.running) or len(prev.entries) > self.token_budget:
            return None
        m = self.manager
        keep = []
        for e in prev.entries:
            r = e.request
            if e.count != 1 or not e.samples or r.finished or r not in self.running:
                return None
            n_out = len(r.output) + 1                      # after prev
            if r.params.max_tokens <= 0 or n_out >= r.params.max_tokens or len(r.prompt) + n_out >= self.max_model_len:
                continue                                   # prev is its last step
            keep.append(e)
        if not keep:
            return None
        needed = [0] * len(m.paged_groups)                 # pages of every group, for all of them together
        for e in keep:
            for gi, n in enumerate(m.pages_missing(e.request.request_id, e.start + 2)):
                needed[gi] += n
        if any(n > g.pool.num_free for n, g in zip(needed, m.paged_groups)):
            return None
        plan = StepPlan()
        for e in keep:
            for g in m.paged_groups:                       # the pools hold them all: counted above
                g.grow(e.request.request_id, e.start + 2)
            plan.entries.append(PlannedEntry(e.request, e.start + 1, 1, True))
        return plan

    def schedule_after_preemption(self, earlier: StepPlan) -> StepPlan:
        plan = self.schedule()
        plan.preempted = earlier.preempted + plan.preempted
        plan.refused = earlier.refused + plan.refused
        plan.truncated = earlier.truncated + plan.truncated
        return plan

    def _keys(self, r: Request) -> list:
        """Keys of the full pages of the request's tokens (made once, continued as the tokens grow)."""
        if self.manager.prefix_reuse:
            r.page_keys = self.manager.page_keys(r.tokens, r.page_keys)
        return r.page_keys

    def _plan_portion(self, r: Request, budget: int, plan: StepPlan) -> int:
        """Give ``r`` as many of its remaining tokens as budget and free pages allow."""
        m = self.manager
        count = min(r.remaining, budget)
        while count > 0 and not m.can_grow(r.request_id, r.computed + count):
            # cut the portion to what the free pages hold
            fits = min(g.pool.num_free + len(g.tables[r.request_id]) for g in m.paged_groups) * m.page_size
            count = min(count - 1, max(0, fits - r.computed))
        if count <= 0:
            return 0
        m.grow(r.request_id, r.computed + count)
        plan.entries.append(PlannedEntry(r, r.computed, count, count == r.remaining))
        return count

    # ------------------------------------------------------------------ after the step
    def commit(self, plan: StepPlan, sampled: Sequence[int], eos_token_ids: Sequence[int] = ()) -> list[Request]:
        """Record the step: ``sampled`` holds one token for each entry with ``samples``,
        in order.  Returns the requests that got a token (finished ones included)."""
        it = iter(sampled)
        touched = []
        m = self.manager
        for e in plan.entries:
            r = e.request
            if r.finished:          # stopped (or aborted) after this step was planned ahead: its token is dropped
                if e.samples:
                    next(it, None)
                continue
            r.computed = e.start + e.count
            if m.prefix_reuse and r.computed // m.page_size > r.published:
                # a page of this request has become full: it is known from now on, not only when the request ends
                m.publish(r.request_id, self._keys(r), r.computed)
                r.published = r.computed // m.page_size
            if not e.samples:
                continue
            tok = int(next(it))
            touched.append(r)
            if r.params.max_tokens <= 0:
                self._finish(r, "length")
                continue
            r.output.append(tok)
            if tok in r.params.stop_token_ids or (tok in eos_token_ids and not r.params.ignore_eos):
                self._finish(r, "stop")
            elif len(r.output) >= r.params.max_tokens:
                self._finish(r, "length")
            elif len(r.prompt) + len(r.output) >= self.max_model_len:
                self._finish(r, "length")
        return touched

    def finish(self, r: Request, reason: str) -> None:
        """End a request for a reason that the engine finds (a stop string in its text)."""
        if not r.finished:
            self._finish(r, reason)

    def fail(self, requests: Sequence[Request], reason: str = "error") -> list[Request]:
        """End the requests of a step that failed.  Their pages go back *unpublished*: what the step wrote may be
        incomplete, so none of it may become known to later requests (pages that earlier, good steps of the same
        request published stay known).  Requests that wait, and running ones that are not named, are untouched
        (acvram/engine/runner.py:1329-1338).  Returns the requests it ended."""
        ended = []
        for r in requests:
            if r.finished or r in ended:
                continue
            r.finished, r.finish_reason = True, reason
            if r in self.running:
                self.running.remove(r)
                self.manager.release(r.request_id)          # no keys: nothing is published on the way out
            elif r in self.waiting:
                self.waiting.remove(r)
            ended.append(r)
        self.counters["failed"] += len(ended)
        return ended

    # ------------------------------------------------------------------ internals
    def _finish(self, r: Request, reason: str) -> None:
        r.finished, r.finish_reason = True, reason
        if r in self.running:
            self.running.remove(r)
            self.manager.release(r.request_id, self._keys(r))

    def _preempt(self, r: Request, plan: StepPlan) -> None:
        self.running.remove(r)
        self.manager.release(r.request_id, self._keys(r))
        plan.entries = [e for e in plan.entries if e.request is not r]
        r.computed = 0
        r.admitted_at = -1
        r.preemptions += 1
        self.waiting.appendleft(r)
        plan.preempted.append(r)
        self.counters["preempted"] += 1
