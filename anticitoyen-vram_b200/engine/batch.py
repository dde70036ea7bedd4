"""The input of one step: a flat batch of (request, its next tokens).

The reference's ``ForwardBatch`` (acvram/engine/lot.py:17-63) carries tokens,
positions, sequence lengths, query lengths, block tables and a slot mapping, and
is either all-prefill or all-decode.  Here a batch mixes portions of prompts and
single decoded tokens freely; per token it gives the token id, its absolute
position and the index of its request in the batch, per request the start of its
tokens, the length of its context after the step, its row of the block tables
and its state slots.  The slot of a token's key and value is computed in the
kernel from the block table (page = table[row][pos // page_size], row in the page
= pos % page_size; acvram/engine/runner.py:1853-1854 has the same arithmetic on
the host).

The block tables themselves stay on the device (``CacheStorage.tables``); a step
brings only the entries that changed since the step before (the reference
rebuilds and copies a padded table every step, acvram/engine/lot.py:98-118).
Everything a step brings is packed into one pinned int32 buffer and reaches the
device with one copy.

What a particular kind of mixer needs beside this (work lists of its kernels,
say) is not made here: a mixer class may offer ``step_metadata`` and
``decode_metadata`` (``parts.base.Mixer``); the builder calls each distinct
provider once a step, packs its arrays into the same buffer and hands the device
views back under the provider's key in ``StepContext.work``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Mapping, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, PagedGroup
from ..kernels import ops


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are asked for


@dataclass
class StepContext:
    num_tokens: int
    num_seqs: int
    num_logit_rows: int
    tokens: torch.Tensor          # int32 [T]
    positions: torch.Tensor       # int32 [T] absolute position of each token in its request
    seq_of_token: torch.Tensor    # int32 [T] index of the token's request in this batch
    cu_q: torch.Tensor            # int32 [B+1] start of each request's tokens in the flat batch
    kv_len: torch.Tensor          # int32 [B] length of each request's context after this step
    logit_rows: torch.Tensor      # int32 [R] rows of the flat batch whose logits are wanted
    table_rows: torch.Tensor | None = None    # int32 [B] each request's row of the block tables (None: its index)
    block_tables: dict[int, torch.Tensor] = field(default_factory=dict)   # group -> int32 [rows, W], kept on the device
    state_slots: dict[int, torch.Tensor] = field(default_factory=dict)    # group -> int32 [B]
    requests: list = field(default_factory=list)
    q_lens: list[int] = field(default_factory=list)
    kv_lens: list[int] = field(default_factory=list)
    work: dict = field(default_factory=dict)   # provider key -> what that kind of mixer asked for (device views, counts)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens, default=0)


def _round4(n: int) -> int:
    return (n + 3) & ~3


class BatchBuilder:
    """Builds StepContexts for one cache manager on one device, reusing its staging buffers."""

    def __init__(self, manager: CacheManager, storage, device, vocab_size: int, max_positions: int,
                 providers: Mapping[str, object] | None = None) -> None:
        self.manager = manager
        self.storage = storage
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self.providers = dict(providers or {})     # key -> object with step_metadata / decode_metadata
        self._paged = [(gi, g) for gi, g in enumerate(manager.groups) if isinstance(g, PagedGroup)]
        # Two pinned staging buffers used in turn: the copy of step n may still be queued
        # on the stream while step n+1 is packed, so a buffer is rewritten only after the
        # event recorded behind its last copy has passed.
        self._hosts: list[torch.Tensor | None] = [None, None]
        self._events: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0
        self.last_h2d_bytes = 0
        self.last_table_updates = 0
        self._dev: torch.Tensor | None = None

    def _buffers(self, n: int) -> tuple[torch.Tensor, torch.Tensor]:
        self._turn ^= 1
        i = self._turn
        cuda = self.device.type == "cuda"
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self._hosts[i] is None or self._hosts[i].numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            self._hosts[i] = torch.empty(cap, dtype=torch.int32, pin_memory=cuda)
        if self._dev is None or self._dev.numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._hosts[i], self._dev

    def _sent(self) -> None:
        if self.device.type == "cuda":
            if self._events[self._turn] is None:
                self._events[self._turn] = torch.cuda.Event()
            self._events[self._turn].record()

    def validate(self, entries: Sequence[StepEntry]) -> None:
        """Refuse a malformed batch before anything is reserved for it."""
        seen = set()
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request!r}: an entry without tokens")
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab_size:
                raise ValueError(f"request {e.request!r}: token id outside the vocabulary of {self.vocab_size}")
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")

    def _apply_updates(self, views: Sequence[tuple[int, torch.Tensor, int]]) -> None:
        """Write the changed block-table entries (already on the device as triples) into the tables."""
        for gi, triples, n in views:
            if n:
                table = self.storage.tables[gi]
                ops.table_update(table, triples, n)

    # ------------------------------------------------------------------ fixed-shape decode batches
    def decode_layout(self, padded: int) -> tuple[dict[str, tuple[int, int]], int, int]:
        """Offsets of the sections of a decode batch padded to ``padded`` rows: first what every step of that
        shape brings anew (tokens, positions, context lengths, rows of the block tables, changed table entries),
        then what is the same for all of them and is written once, when the shape's graph is captured.
        Returns (offsets, ints a step brings, ints in all)."""
        off, out = 0, {}
        dynamic = [("tokens", padded), ("positions", padded), ("kv_len", padded), ("table_rows", padded),
                   *[(f"st{gi}", padded) for gi, g in enumerate(self.manager.groups) if not isinstance(g, PagedGroup)],
                   *[(f"upd{gi}", 3 * 2 * padded) for gi, _ in self._paged]]
        for name, n in dynamic:
            out[name] = (off, n)
            off += _round4(n)
        n_dynamic = off
        static = [("seq_of_token", padded), ("cu_q", padded + 1), ("logit_rows", padded)]
        for key, prov in self.providers.items():
            meta = prov.decode_metadata(padded, 1)
            static += [(f"{key}.{name}", int(np.asarray(a).size)) for name, a in meta.arrays.items()]
        for name, n in static:
            out[name] = (off, n)
            off += _round4(n)
        return out, n_dynamic, off

    def build_decode(self, entries: Sequence[StepEntry], starts: Sequence[int], padded: int, max_kv: int,
                     dev: torch.Tensor, first: bool = False) -> StepContext:
        """One token for each request, padded to ``padded`` rows (padding rows hold nothing: context
        length 0 and the block tables' row that belongs to nobody, so they read and write no page), into the
        buffer ``dev``.  ``max_kv``: the context length that the launch shapes of this bucket are made for.
        ``first``: also write the part that never changes (at capture)."""
        m = self.manager
        B = len(entries)
        layout, n_dynamic, total = self.decode_layout(padded)
        host, _ = self._buffers(total)
        h = host.numpy()

        def put(name, values, fill=0):
            o, n = layout[name]
            h[o:o + n] = fill
            h[o:o + len(values)] = values

        put("tokens", [e.tokens[0] for e in entries])
        put("positions", list(starts))
        put("kv_len", [s + 1 for s in starts])
        put("table_rows", [m.rows[e.request] for e in entries], fill=m.null_row)
        last_fixed = "table_rows"
        for gi, g in enumerate(m.groups):
            if not isinstance(g, PagedGroup):      # padding rows work on the state slot that belongs to nobody
                put(f"st{gi}", [g.slot_of[e.request] for e in entries], fill=g.max_requests)
                last_fixed = f"st{gi}"
        updates = m.take_updates()
        late = []      # more changed entries than the fixed section holds (rare: sent by themselves)
        views = []
        self.last_table_updates = sum(len(u) for u in updates)
        for (gi, _), upd in zip(self._paged, updates):
            o, n = layout[f"upd{gi}"]
            if 3 * len(upd) > n:
                late.append((gi, upd))
                continue
            if upd:
                h[o:o + 3 * len(upd)] = np.asarray(upd, dtype=np.int32).reshape(-1)
            views.append((gi, dev[o:o + n], len(upd)))
        metas = {}
        if first:
            ar = np.arange(padded + 1, dtype=np.int32)
            put("seq_of_token", ar[:padded])
            put("cu_q", ar)
            put("logit_rows", ar[:padded])
        for key, prov in self.providers.items():
            metas[key] = prov.decode_metadata(padded, max_kv)
            if first:
                for name, a in metas[key].arrays.items():
                    put(f"{key}.{name}", np.asarray(a, dtype=np.int32).reshape(-1))
        # a step sends what it brings: up to the end of the last changed table entry (the rest of the buffer is static)
        n_send = layout[last_fixed][0] + _round4(padded)
        for gi, _, n_upd in views:
            if n_upd:
                n_send = max(n_send, layout[f"upd{gi}"][0] + _round4(3 * n_upd))
        if first:
            n_send = total
        dev[:n_send].copy_(host[:n_send], non_blocking=True)
        self.last_h2d_bytes = n_send * 4
        self._sent()
        for gi, upd in late:
            t = torch.tensor(upd, dtype=torch.int32).reshape(-1).to(self.device)
            self.last_h2d_bytes += t.numel() * 4
            views.append((gi, t, len(upd)))
        self._apply_updates(views)

        view = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
        kv_lens = [s + 1 for s in starts]
        ctx = StepContext(
            num_tokens=padded, num_seqs=padded, num_logit_rows=padded, tokens=view("tokens"),
            positions=view("positions"), seq_of_token=view("seq_of_token"), cu_q=view("cu_q"), kv_len=view("kv_len"),
            logit_rows=view("logit_rows"), table_rows=view("table_rows"), requests=[e.request for e in entries],
            q_lens=[1] * padded, kv_lens=kv_lens + [0] * (padded - B))
        for gi, g in enumerate(m.groups):
            if isinstance(g, PagedGroup):
                ctx.block_tables[gi] = self.storage.tables[gi]
            else:
                ctx.state_slots[gi] = view(f"st{gi}")
        for key, meta in metas.items():
            ctx.work[key] = {**{name: view(f"{key}.{name}") for name in meta.arrays}, **meta.values}
        return ctx

    # ------------------------------------------------------------------ any batch
    def build(self, entries: Sequence[StepEntry], starts: Sequence[int]) -> StepContext:
        """``starts[i]`` is the number of tokens request i held before this step; its pages
        for the new tokens are already reserved."""
        m = self.manager
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        T = sum(q_lens)
        if any(q == 0 for q in q_lens):
            raise ValueError("an entry without tokens")
        kv_lens = [s + q for s, q in zip(starts, q_lens)]
        if max(kv_lens, default=0) > self.max_positions:
            raise ValueError(f"a request would reach {max(kv_lens)} tokens; the model has {self.max_positions} positions")

        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]) if B else np.zeros(0, np.int64)
        if T and (tokens.min() < 0 or tokens.max() >= self.vocab_size):
            raise ValueError(f"token id outside the vocabulary of {self.vocab_size}")
        cu = np.zeros(B + 1, dtype=np.int32)
        np.cumsum(q_lens, out=cu[1:])
        seq_of = np.repeat(np.arange(B, dtype=np.int32), q_lens)
        positions = np.arange(T, dtype=np.int32) - np.repeat(cu[:-1] - np.asarray(starts, dtype=np.int32), q_lens)
        rows = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < q_lens[i]:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {q_lens[i]} tokens")
                rows.append(int(cu[i]) + int(w))
        R = len(rows)

        sections: list[tuple[str, np.ndarray]] = [
            ("tokens", tokens.astype(np.int32)), ("positions", positions), ("seq_of_token", seq_of), ("cu_q", cu),
            ("kv_len", np.asarray(kv_lens, dtype=np.int32)), ("logit_rows", np.asarray(rows, dtype=np.int32)),
            ("table_rows", np.asarray([m.rows[e.request] for e in entries], dtype=np.int32))]
        for gi, g in enumerate(m.groups):
            if not isinstance(g, PagedGroup):
                sections.append((f"st{gi}", np.asarray([g.slot_of[e.request] for e in entries], dtype=np.int32)))
        updates = m.take_updates()
        self.last_table_updates = sum(len(u) for u in updates)
        for (gi, _), upd in zip(self._paged, updates):
            sections.append((f"upd{gi}", np.asarray(upd, dtype=np.int32).reshape(-1)))
        metas = {key: prov.step_metadata(q_lens, kv_lens, cu) for key, prov in self.providers.items()}
        for key, meta in metas.items():
            for name, a in meta.arrays.items():
                sections.append((f"{key}.{name}", np.ascontiguousarray(a, dtype=np.int32).reshape(-1)))

        total = sum(_round4(a.size) for _, a in sections)
        host, dev = self._buffers(max(total, 4))
        hnp = host.numpy()
        offsets = {}
        off = 0
        for name, arr in sections:
            hnp[off:off + arr.size] = arr
            offsets[name] = (off, arr.size)
            off += _round4(arr.size)
        dev[:total].copy_(host[:total], non_blocking=True)
        self.last_h2d_bytes = total * 4
        self._sent()

        def view(name: str) -> torch.Tensor:
            o, n = offsets[name]
            return dev[o:o + n]

        self._apply_updates([(gi, view(f"upd{gi}"), len(upd)) for (gi, _), upd in zip(self._paged, updates)])
        ctx = StepContext(
            num_tokens=T, num_seqs=B, num_logit_rows=R, tokens=view("tokens"), positions=view("positions"),
            seq_of_token=view("seq_of_token"), cu_q=view("cu_q"), kv_len=view("kv_len"), logit_rows=view("logit_rows"),
            table_rows=view("table_rows"), requests=[e.request for e in entries], q_lens=q_lens, kv_lens=kv_lens)
        for gi, g in enumerate(m.groups):
            if isinstance(g, PagedGroup):
                ctx.block_tables[gi] = self.storage.tables[gi]
            else:
                ctx.state_slots[gi] = view(f"st{gi}")
        for key, meta in metas.items():
            ctx.work[key] = {**{name: view(f"{key}.{name}") for name in meta.arrays}, **meta.values}
        return ctx
