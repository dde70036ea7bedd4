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
ends, 1771-1803) plus the window rule above.

Prefix reuse, as the reference's allocator has it (reference counts, a chained
hash over the tokens of each full page, freed-but-known pages kept until their
room is needed; acvram/memory/kvcache.py:100-165): when a request ends, its full
pages are *published* under the hash of all tokens up to and including theirs; a
later request whose tokens begin the same way takes those pages into its block
table instead of computing them again, and several requests may hold one page.
Shared pages are never written: a request writes only at positions past what it
holds.  Reuse is switched on by ``enable_prefix_cache`` and needs every group to
keep all keys (a window gives pages back as it goes, and a state of fixed size
has no page to take over).

The block tables also live on the device, one row for each live request, and
stay there between steps (the reference rebuilds a padded table on the host and
copies it every step, acvram/engine/lot.py:98-118).  The manager gives every
request a *row* when it is admitted and notes each entry that changes (a page
reserved, taken over, or given back by a window); ``take_updates`` hands those
(row, column, page) triples to the step that is being built, which sends them
along with its tokens.

This file is host-side bookkeeping only and imports no torch at module level;
``CacheStorage`` holds the tensors.
"""

from __future__ import annotations

import hashlib
from array import array
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Hashable, Sequence


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

    @property
    def takes_over(self) -> bool:
        """Whether a new request can start on pages that an earlier request filled: yes where all keys are kept
        (a window gives pages back as it goes, so an earlier request's first pages are gone)."""
        return self.window <= 0


@dataclass(frozen=True)
class StateNeed:
    shape: tuple[int, ...]
    dtype: str = "float32"

    @property
    def kind(self) -> str:
        return "state"

    @property
    def takes_over(self) -> bool:
        """A state of fixed size has no page to hand to a later request; a mixer that wanted to join prefix reuse
        would have to keep a copy of its state at every page's end (the hook is not built: no part here needs it)."""
        return False


class PagePool:
    """Page numbers ``0 .. num_pages-1``, each one free, held (by one or more block tables) or *kept*:
    held by nobody, but still filled with published content that a later request may take over.
    Free pages are given out first, last freed first reused; then kept pages, the longest unused first."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._refs = [0] * num_pages
        self._key: list[bytes | None] = [None] * num_pages      # the content a page is published under
        self._index: dict[bytes, int] = {}                      # published content -> page
        self._kept: OrderedDict[int, None] = OrderedDict()      # published pages that nobody holds, oldest first

    @property
    def num_free(self) -> int:
        """Pages that ``allocate`` can give: the free ones and the kept ones."""
        return len(self._free) + len(self._kept)

    @property
    def num_kept(self) -> int:
        return len(self._kept)

    def allocate(self, n: int) -> list[int]:
        if n > self.num_free:
            raise OutOfPages(f"{n} pages asked, {self.num_free} free of {self.num_pages}")
        out = []
        for _ in range(n):
            if self._free:
                p = self._free.pop()
            else:                               # the room of the page that went unused longest
                p, _ = self._kept.popitem(last=False)
                del self._index[self._key[p]]
                self._key[p] = None
            self._refs[p] = 1
            out.append(p)
        return out

    def release(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages or self._refs[p] <= 0:
                raise CacheAccountingError(f"page {p} is released but not held")
            self._refs[p] -= 1
            if self._refs[p] == 0:
                if self._key[p] is not None:
                    self._kept[p] = None
                else:
                    self._free.append(p)

    # ---- published content
    def publish(self, page: int, key: bytes) -> None:
        """``page`` (held) is full of the content named ``key``; a second page of the same content stays unnamed."""
        if not 0 <= page < self.num_pages or self._refs[page] <= 0:
            raise CacheAccountingError(f"page {page} is published but not held")
        if self._key[page] is None and key not in self._index:
            self._key[page] = key
            self._index[key] = page

    def lookup(self, key: bytes) -> int | None:
        return self._index.get(key)

    def is_kept(self, page: int) -> bool:
        return page in self._kept

    def share(self, page: int) -> None:
        """One more holder of a published page (held by others, or kept)."""
        if self._key[page] is None or (self._refs[page] == 0 and page not in self._kept):
            raise CacheAccountingError(f"page {page} is shared but holds no published content")
        self._kept.pop(page, None)
        self._refs[page] += 1

    def holders(self, page: int) -> int:
        return self._refs[page]

    def check(self) -> None:
        """Every page is free, kept or held, and only one of them; the index names published pages only."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheAccountingError("a page is on the free list twice")
        for p in range(self.num_pages):
            states = (p in free) + (p in self._kept) + (self._refs[p] > 0)
            if states != 1:
                raise CacheAccountingError(f"page {p} is {'lost' if states == 0 else 'in two states at once'}")
            if (p in free or p in self._kept) and self._refs[p] != 0:
                raise CacheAccountingError(f"page {p} is counted as held and is not")
            if p in self._kept and self._key[p] is None:
                raise CacheAccountingError(f"page {p} is kept without content")
            if p in free and self._key[p] is not None:
                raise CacheAccountingError(f"page {p} is free and still published")
        for key, p in self._index.items():
            if self._key[p] != key:
                raise CacheAccountingError(f"the index names page {p} under content it does not hold")
        if sum(k is not None for k in self._key) != len(self._index):
            raise CacheAccountingError("published pages and index entries do not add up")


class PagedGroup:
    """Cache slots with the same ``PagedNeed``: one pool, one block table per request."""

    def __init__(self, need: PagedNeed, num_slots: int, page_size: int, num_pages: int) -> None:
        self.need = need
        self.num_slots = num_slots
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.tables: dict[Hashable, list[int]] = {}
        self.first_live: dict[Hashable, int] = {}  # first page index not yet released by the window
        self.rows: dict[Hashable, int] = {}        # request -> its row of the device table (the manager's dict)
        self.dirty: list[tuple[int, int, int]] = []   # (row, column, page) entries that the device table lacks

    def _note(self, request, first_col: int, pages) -> None:
        row = self.rows.get(request)
        if row is not None:
            self.dirty.extend((row, first_col + i, p) for i, p in enumerate(pages))

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def missing(self, request, length: int) -> int:
        return max(0, self.pages_for(length) - len(self.tables[request]))

    def grow(self, request, length: int) -> None:
        n = self.missing(request, length)
        if n:
            self.extend(request, self.pool.allocate(n))

    def extend(self, request, pages: Sequence[int]) -> None:
        table = self.tables[request]
        self._note(request, len(table), pages)
        table.extend(pages)

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
            self._note(request, start, [-1] * len(freed))
            self.pool.release(freed)
            self.first_live[request] = releasable
        return len(freed)

    def set_page(self, request, index: int, page: int) -> None:
        """Put ``page`` at ``index`` of the request's block table (the books of the pool are the caller's to keep:
        tests use it to make a table wrong on purpose)."""
        self.tables[request][index] = page
        self._note(request, index, [page])

    def drop(self, request) -> None:
        table = self.tables.pop(request)
        self.first_live.pop(request)
        # the last page first: of a chain of kept pages the deepest is then the first to lose its room,
        # and the pages before it stay reachable
        self.pool.release([p for p in reversed(table) if p >= 0])

    # ---- prefix reuse
    def matching(self, keys: Sequence[bytes]) -> list[int]:
        """The pages published under the leading ``keys``, up to the first that is not there."""
        pages = []
        for key in keys:
            p = self.pool.lookup(key)
            if p is None:
                break
            pages.append(p)
        return pages

    def adopt(self, request, pages: Sequence[int]) -> None:
        """A new request's block table begins with published pages."""
        for p in pages:
            self.pool.share(p)
        self.tables[request] = list(pages)
        self._note(request, 0, pages)

    def publish(self, request, keys: Sequence[bytes]) -> None:
        for p, key in zip(self.tables[request], keys):
            if p >= 0:
                self.pool.publish(p, key)


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

    def __init__(self, plan: CachePlan, page_size: int, num_pages: int | list[int], max_requests: int,
                 enable_prefix_cache: bool = False) -> None:
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
        self._paged = [g for g in self.groups if isinstance(g, PagedGroup)]      # the groups never change
        self._state = [g for g in self.groups if isinstance(g, StateGroup)]
        self.lengths: dict[Hashable, int] = {}
        # rows of the device block tables: one for each live request, the same in every group; row
        # ``max_requests`` belongs to nobody and stays at -1 (padding rows of a fixed-shape batch point there)
        self.rows: dict[Hashable, int] = {}
        self._free_rows = list(range(max_requests - 1, -1, -1))
        for g in self._paged:
            g.rows = self.rows
        # pages are taken over only where every group keeps all keys in pages
        # (every group is asked: each need says whether what it keeps can be handed to a later request)
        self.prefix_reuse = bool(enable_prefix_cache) and bool(self.groups) and all(g.need.takes_over for g in self.groups)
        self.reused_tokens = 0          # tokens that requests took over instead of computing them

    # ------------------------------------------------------------------ prefix reuse
    def page_keys(self, tokens: Sequence[int], known: Sequence[bytes] = ()) -> list[bytes]:
        """One key for each full page of ``tokens``: a hash of all tokens up to the page's end, chained
        from page to page (the reference chains its hashes the same way, acvram/memory/kvcache.py:153-165).
        ``known``: the keys of the first pages, from an earlier call with a beginning of the same tokens."""
        ps = self.page_size
        keys = list(known[:len(tokens) // ps])
        parent = keys[-1] if keys else b""
        for i in range(len(keys), len(tokens) // ps):
            parent = hashlib.blake2b(parent + array("q", tokens[i * ps:(i + 1) * ps]).tobytes(), digest_size=16).digest()
            keys.append(parent)
        return keys

    def reusable(self, keys: Sequence[bytes], num_tokens: int) -> tuple[int, list[int]]:
        """(tokens, kept pages of each group among them) that a new request of ``num_tokens`` tokens, whose
        full pages have the ``keys``, would take over.

        At least the last token is left to be computed: its logits are what the request is admitted for."""
        if not self.prefix_reuse or num_tokens < 2:
            return 0, [0] * len(self.paged_groups)
        keys = keys[:(num_tokens - 1) // self.page_size]
        found = [g.matching(keys) for g in self.paged_groups]
        n = min(len(f) for f in found)
        return n * self.page_size, [sum(g.pool.is_kept(p) for p in f[:n]) for g, f in zip(self.paged_groups, found)]

    def can_admit_with(self, keys: Sequence[bytes], num_tokens: int, first: int) -> bool:
        """Whether the pools hold the first ``first`` new tokens of such a request beside the published
        pages that it takes over (which leave the kept ones and stop counting as free)."""
        reuse, kept = self.reusable(keys, num_tokens)
        return all(g.pages_for(reuse + first) - reuse // self.page_size <= g.pool.num_free - k
                   for g, k in zip(self.paged_groups, kept))

    # ------------------------------------------------------------------ queries
    @property
    def paged_groups(self) -> list[PagedGroup]:
        return self._paged

    @property
    def state_groups(self) -> list[StateGroup]:
        return self._state

    def live(self) -> list:
        return list(self.lengths)

    def can_admit(self) -> bool:
        return len(self.lengths) < self.max_requests and all(g.num_free > 0 for g in self.state_groups)

    def pages_missing(self, request, length: int) -> list[int]:
        """Pages that each paged group still needs so that ``request`` holds ``length`` tokens."""
        return [g.missing(request, length) for g in self.paged_groups]

    def can_grow(self, request, length: int, reserve: list[int] | None = None) -> bool:
        if reserve is None:
            return all(g.missing(request, length) <= g.pool.num_free for g in self._paged)
        return all(g.missing(request, length) + r <= g.pool.num_free for g, r in zip(self._paged, reserve))

    def fits_empty_pool(self, length: int) -> bool:
        """Could a request of ``length`` tokens ever be held, with every page free?

        A windowed group frees pages as it goes, but within one step it may need the whole portion."""
        return all(g.pages_for(length) <= g.pool.num_pages for g in self.paged_groups if g.need.window <= 0)

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.paged_groups]

    # ------------------------------------------------------------------ life of a request
    def admit(self, request, keys: Sequence[bytes] = (), num_tokens: int = 0) -> dict[int, int]:
        """Start a request: empty block tables, one state slot in each state group.

        With the ``keys`` of the full pages of the ``num_tokens`` tokens that the request brings (as far
        as known) and prefix reuse on, the block tables begin with the published pages of the longest
        known beginning, and the request's length starts there (``lengths[request]``).
        Returns {group index: state slot}; the caller zeroes those slots."""
        if request in self.lengths:
            raise CacheAccountingError(f"request {request!r} is admitted twice")
        if not self.can_admit():
            raise OutOfPages("no room for another request")
        slots = {}
        reuse, _ = self.reusable(keys, num_tokens)
        keys = keys[:reuse // self.page_size]
        self.rows[request] = self._free_rows.pop()
        for gi, g in enumerate(self.groups):
            if isinstance(g, PagedGroup):
                g.tables[request] = []
                g.first_live[request] = 0
                if keys:
                    g.adopt(request, g.matching(keys))
            else:
                slots[gi] = g.take(request)
        self.lengths[request] = reuse
        self.reused_tokens += reuse
        return slots

    def grow(self, request, length: int) -> None:
        """Reserve pages so that positions [0, length) exist; all groups or none.

        Reserving does not move the request's length: ``advance`` does, once the
        tokens have run.  Growing to a length already reserved takes nothing."""
        need = [g.missing(request, length) for g in self._paged]
        if any(n > g.pool.num_free for n, g in zip(need, self._paged)):
            raise OutOfPages(f"request {request!r} cannot grow to {length} tokens: free {self.free_pages()}")
        for n, g in zip(need, self._paged):
            if n:
                g.extend(request, g.pool.allocate(n))

    def advance(self, request, length: int) -> None:
        """The request now holds ``length`` tokens in its pages."""
        for g in self.paged_groups:
            if g.pages_for(length) > len(g.tables[request]):
                raise CacheAccountingError(f"request {request!r} advanced to {length} tokens beyond its pages")
        self.lengths[request] = length

    def trim(self, request) -> int:
        """After a step: release what every window has passed.  Returns pages freed."""
        return sum(g.trim(request, self.lengths[request]) for g in self.paged_groups)

    def publish(self, request, keys: Sequence[bytes], num_tokens: int) -> None:
        """The request's pages that positions [0, num_tokens) fill become known under ``keys`` while the
        request goes on (it never writes them again), so that requests admitted meanwhile can take them over."""
        if not self.prefix_reuse:
            return
        keys = keys[:min(num_tokens, self.lengths[request]) // self.page_size]
        for g in self.paged_groups:
            g.publish(request, keys)

    def release(self, request, keys: Sequence[bytes] = ()) -> None:
        """Give back what the request holds.  With the ``keys`` of the full pages of its tokens (from
        position 0) and prefix reuse on, the full pages that it holds are published first."""
        if request not in self.lengths:
            raise CacheAccountingError(f"request {request!r} is released but not live")
        if keys and self.prefix_reuse:
            keys = keys[:self.lengths[request] // self.page_size]
            for g in self.paged_groups:
                g.publish(request, keys)
        for g in self.groups:
            if isinstance(g, PagedGroup):
                g.drop(request)
            else:
                g.give_back(request)
        del self.lengths[request]
        self._free_rows.append(self.rows.pop(request))

    # ------------------------------------------------------------------ the device's copy of the block tables
    @property
    def null_row(self) -> int:
        return self.max_requests

    def take_updates(self) -> list[list[tuple[int, int, int]]]:
        """For each paged group the (row, column, page) entries that changed since the last call, each entry once."""
        out = []
        for g in self._paged:
            # an entry noted twice (a row given back and taken again before a step ran) goes out once, with its last
            # value: the kernel that writes the entries runs them side by side
            last = {(row, col): page for row, col, page in g.dirty}
            out.append([(row, col, page) for (row, col), page in last.items()] if len(last) != len(g.dirty) else g.dirty)
            g.dirty = []
        return out

    def resync(self) -> None:
        """Note every entry of every live request again (after a step failed somewhere between taking the
        updates and sending them, the device's tables cannot be trusted)."""
        for g in self._paged:
            g.dirty = [(self.rows[r], c, p) for r, table in g.tables.items() for c, p in enumerate(table)]

    # ------------------------------------------------------------------ views
    def block_table(self, request, group: int) -> list[int]:
        return self.groups[group].tables[request]

    def state_slot(self, request, group: int) -> int:
        return self.groups[group].slot_of[request]

    def check(self) -> None:
        for g in self.paged_groups:
            g.pool.check()
            held: dict[int, int] = {}
            for table in g.tables.values():
                if len([p for p in table if p >= 0]) != len({p for p in table if p >= 0}):
                    raise CacheAccountingError("a page is in one block table twice")
                for p in table:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p, n in held.items():
                if g.pool.holders(p) != n:
                    raise CacheAccountingError(f"page {p} is in {n} block tables and counted {g.pool.holders(p)} times")
                if n > 1 and not self.prefix_reuse:
                    raise CacheAccountingError("a page is in two block tables")
            if len(held) + g.pool.num_free != g.pool.num_pages:
                raise CacheAccountingError("held + free pages do not add up to the pool")
        for g in self.state_groups:
            if len(set(g.slot_of.values())) != len(g.slot_of) or len(g.slot_of) + g.num_free != g.max_requests:
                raise CacheAccountingError("state slots do not add up")
        if (set(self.rows) != set(self.lengths) or len(set(self.rows.values())) != len(self.rows)
                or sorted(list(self.rows.values()) + self._free_rows) != list(range(self.max_requests))):
            raise CacheAccountingError("rows of the block tables do not add up")
