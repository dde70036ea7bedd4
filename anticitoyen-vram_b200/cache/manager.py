"""The cache manager: pages of keys and values with a block table for each
request, and slots for per-request state of fixed size.

What a mixer keeps for a request is declared as a *need*:

* ``PagedNeed``  - something that grows by one entry for each token (attention's
  keys and values), kept in pages of ``page_size`` tokens; with ``window`` > 0
  only the last ``window`` tokens are ever read again, so older pages go back to
  the pool as soon as the window has passed them.
* ``StateNeed``  - a tensor of fixed shape for each live request (a recurrent
  state), kept in a slot that is given at admission, zeroed, and taken back when
  the request ends.

Cache slots (one for each layer that keeps something) with equal needs form a
*group*; a group has its own pool of pages, its own block tables and its own
device storage, so that layers that keep everything and layers that keep a window
do not share pages.  A page number means the same page in every slot of its
group, as in the reference, where one allocator serves all layers
(acvram/engine/runner.py:795-808); the reference's page is 16 tokens, fixed in
code (acvram/memory/kvcache.py:37), here it is a parameter.

The life of a request's pages follows the reference (pages reserved as the
request grows, acvram/engine/runner.py:1762-1769; all given back at once when it
ends, 1771-1803) plus the window rule above.  This file is host-side bookkeeping
only and imports no torch at module level; ``CacheStorage`` holds the tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable


class OutOfPages(RuntimeError):
    """The pool cannot give the pages asked for; nothing was taken."""


class CacheAccountingError(AssertionError):
    """A page or slot was freed twice, or freed without being held."""


@dataclass(frozen=True)
class PagedNeed:
    num_kv_heads: int
    head_dim: int
    window: int = 0

    @property
    def kind(self) -> str:
        return "paged"


@dataclass(frozen=True)
class StateNeed:
    shape: tuple[int, ...]
    dtype: str = "float32"

    @property
    def kind(self) -> str:
        return "state"


class PagePool:
    """Free list of page numbers ``0 .. num_pages-1``; last freed, first reused."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages asked, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def release(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or not self._held[p]:
                raise CacheAccountingError(f"page {p} is released but not held")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """Every page is either free or held, and none is both or twice free."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheAccountingError("a page is on the free list twice")
        for p in range(self.num_pages):
            if self._held[p] == (p in free):
                raise CacheAccountingError(f"page {p} is {'both held and free' if self._held[p] else 'lost'}")


class PagedGroup:
    """Cache slots with the same ``PagedNeed``: one pool, one block table per request."""

    def __init__(self, need: PagedNeed, num_slots: int, page_size: int, num_pages: int) -> None:
        self.need = need
        self.num_slots = num_slots
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: dict[Hashable, list[int]] = {}
        self.first_live: dict[Hashable, int] = {}  # first page index not yet released by the window

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def missing(self, request, length: int) -> int:
        return max(0, self.pages_for(length) - len(self.tables[request]))

    def grow(self, request, length: int) -> None:
        n = self.missing(request, length)
        if n:
            self.tables[request].extend(self.pool.allocate(n))

    def trim(self, request, kv_len: int) -> int:
        """Give back the pages whose every key is out of the window of any later query."""
        w = self.need.window
        if w <= 0:
            return 0
        table = self.tables[request]
        releasable = max(0, (kv_len - w + 1) // self.page_size)
        releasable = min(releasable, len(table))
        start = self.first_live[request]
        freed = [table[i] for i in range(start, releasable)]
        for i in range(start, releasable):
            table[i] = -1
        if freed:
            self.pool.release(freed)
            self.first_live[request] = releasable
        return len(freed)

    def drop(self, request) -> None:
        table = self.tables.pop(request)
        self.first_live.pop(request)
        self.pool.release([p for p in table if p >= 0])


class StateGroup:
    """Cache slots with the same ``StateNeed``: one state slot per live request."""

    def __init__(self, need: StateNeed, num_slots: int, max_requests: int) -> None:
        self.need = need
        self.num_slots = num_slots
        self.max_requests = max_requests
        self._free = list(range(max_requests - 1, -1, -1))
        self.slot_of: dict[Hashable, int] = {}

    def take(self, request) -> int:
        if not self._free:
            raise OutOfPages(f"no state slot free of {self.max_requests}")
        slot = self._free.pop()
        self.slot_of[request] = slot
        return slot

    def give_back(self, request) -> None:
        slot = self.slot_of.pop(request, None)
        if slot is None or slot in self._free:
            raise CacheAccountingError(f"state slot of {request!r} is released but not held")
        self._free.append(slot)

    @property
    def num_free(self) -> int:
        return len(self._free)


@dataclass
class CachePlan:
    """Which cache slot belongs to which group: the model's answer to 'what do you keep?'."""

    needs: list  # one need (PagedNeed | StateNeed | None) for each cache slot of the model
    groups: list = field(default_factory=list)  # distinct needs, in order of first appearance
    group_of_slot: list[int] = field(default_factory=list)  # cache slot -> group index (-1: keeps nothing)
    index_in_group: list[int] = field(default_factory=list)  # cache slot -> position inside its group

    def __post_init__(self) -> None:
        counts: list[int] = []
        for need in self.needs:
            if need is None:
                self.group_of_slot.append(-1)
                self.index_in_group.append(-1)
                continue
            if need not in self.groups:
                self.groups.append(need)
                counts.append(0)
            g = self.groups.index(need)
            self.group_of_slot.append(g)
            self.index_in_group.append(counts[g])
            counts[g] += 1
        self.slots_per_group = counts


class CacheManager:
    """Pages and state slots of all live requests, for all groups."""

    def __init__(self, plan: CachePlan, page_size: int, num_pages: int | list[int], max_requests: int) -> None:
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.plan = plan
        self.page_size = page_size
        self.max_requests = max_requests
        per_group = num_pages if isinstance(num_pages, (list, tuple)) else [num_pages] * len(plan.groups)
        self.groups: list[PagedGroup | StateGroup] = []
        for need, n_slots, n_pages in zip(plan.groups, plan.slots_per_group, per_group):
            if need.kind == "paged":
                self.groups.append(PagedGroup(need, n_slots, page_size, n_pages))
            else:
                self.groups.append(StateGroup(need, n_slots, max_requests))
        self.lengths: dict[Hashable, int] = {}

    # ------------------------------------------------------------------ queries
    @property
    def paged_groups(self) -> list[PagedGroup]:
        return [g for g in self.groups if isinstance(g, PagedGroup)]

    @property
    def state_groups(self) -> list[StateGroup]:
        return [g for g in self.groups if isinstance(g, StateGroup)]

    def live(self) -> list:
        return list(self.lengths)

    def can_admit(self) -> bool:
        return len(self.lengths) < self.max_requests and all(g.num_free > 0 for g in self.state_groups)

    def pages_missing(self, request, length: int) -> list[int]:
        """Pages that each paged group still needs so that ``request`` holds ``length`` tokens."""
        return [g.missing(request, length) for g in self.paged_groups]

    def can_grow(self, request, length: int, reserve: list[int] | None = None) -> bool:
        reserve = reserve or [0] * len(self.paged_groups)
        return all(g.missing(request, length) + r <= g.pool.num_free for g, r in zip(self.paged_groups, reserve))

    def fits_empty_pool(self, length: int) -> bool:
        """Could a request of ``length`` tokens ever be held, with every page free?

        A windowed group frees pages as it goes, but within one step it may need the whole portion."""
        return all(g.pages_for(length) <= g.pool.num_pages for g in self.paged_groups if g.need.window <= 0)

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.paged_groups]

    # ------------------------------------------------------------------ life of a request
    def admit(self, request) -> dict[int, int]:
        """Start a request: empty block tables, one state slot in each state group.

        Returns {group index: state slot}; the caller zeroes those slots."""
        if request in self.lengths:
            raise CacheAccountingError(f"request {request!r} is admitted twice")
        if not self.can_admit():
            raise OutOfPages("no room for another request")
        slots = {}
        for gi, g in enumerate(self.groups):
            if isinstance(g, PagedGroup):
                g.tables[request] = []
                g.first_live[request] = 0
            else:
                slots[gi] = g.take(request)
        self.lengths[request] = 0
        return slots

    def grow(self, request, length: int) -> None:
        """Reserve pages so that positions [0, length) exist; all groups or none.

        Reserving does not move the request's length: ``advance`` does, once the
        tokens have run.  Growing to a length already reserved takes nothing."""
        if not self.can_grow(request, length):
            raise OutOfPages(f"request {request!r} cannot grow to {length} tokens: free {self.free_pages()}")
        for g in self.paged_groups:
            g.grow(request, length)

    def advance(self, request, length: int) -> None:
        """The request now holds ``length`` tokens in its pages."""
        for g in self.paged_groups:
            if g.pages_for(length) > len(g.tables[request]):
                raise CacheAccountingError(f"request {request!r} advanced to {length} tokens beyond its pages")
        self.lengths[request] = length

    def trim(self, request) -> int:
        """After a step: release what every window has passed.  Returns pages freed."""
        return sum(g.trim(request, self.lengths[request]) for g in self.paged_groups)

    def release(self, request) -> None:
        if request not in self.lengths:
            raise CacheAccountingError(f"request {request!r} is released but not live")
        for g in self.groups:
            if isinstance(g, PagedGroup):
                g.drop(request)
            else:
                g.give_back(request)
        del self.lengths[request]

    # ------------------------------------------------------------------ views
    def block_table(self, request, group: int) -> list[int]:
        return self.groups[group].tables[request]

    def state_slot(self, request, group: int) -> int:
        return self.groups[group].slot_of[request]

    def check(self) -> None:
        for g in self.paged_groups:
            g.pool.check()
            held = [p for table in g.tables.values() for p in table if p >= 0]
            if len(held) != len(set(held)):
                raise CacheAccountingError("a page is in two block tables")
            if len(held) + g.pool.num_free != g.pool.num_pages:
                raise CacheAccountingError("held + free pages do not add up to the pool")
        for g in self.state_groups:
            if len(set(g.slot_of.values())) != len(g.slot_of) or len(g.slot_of) + g.num_free != g.max_requests:
                raise CacheAccountingError("state slots do not add up")
