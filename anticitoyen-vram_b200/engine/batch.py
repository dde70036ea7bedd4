"""The input of one step: a flat batch of (request, its next tokens).

The reference's ``ForwardBatch`` (acvram/engine/lot.py:17-63) carries tokens,
positions, sequence lengths, query lengths, block tables and a slot mapping, and
is either all-prefill or all-decode.  Here a batch mixes portions of prompts and
single decoded tokens freely; per token it gives the token id, its absolute
position and the index of its request in the batch, per request the start of its
tokens, the length of its context after the step, its row of each group's block
table and its state slots.  The slot of a token's key and value is computed in
the kernel from the block table (page = table[pos // page_size], row = pos %
page_size; acvram/engine/runner.py:1853-1854 has the same arithmetic on the host).

Everything is packed into one pinned int32 buffer and reaches the device with one
copy per step.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, PagedGroup


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
    block_tables: dict[int, torch.Tensor] = field(default_factory=dict)   # group -> int32 [B, W]
    state_slots: dict[int, torch.Tensor] = field(default_factory=dict)    # group -> int32 [B]
    requests: list = field(default_factory=list)
    q_lens: list[int] = field(default_factory=list)
    kv_lens: list[int] = field(default_factory=list)
    work: dict = field(default_factory=dict)   # per-step work lists of the attention kernels (device views)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens, default=0)


QUERY_TILE = 128   # query tokens per tile of the portion-attention kernels


def _round4(n: int) -> int:
    return (n + 3) & ~3


class BatchBuilder:
    """Builds StepContexts for one cache manager on one device, reusing its staging buffers."""

    def __init__(self, manager: CacheManager, device, vocab_size: int, max_positions: int) -> None:
        self.manager = manager
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        # Two pinned staging buffers used in turn: the copy of step n may still be queued
        # on the stream while step n+1 is packed, so a buffer is rewritten only after the
        # event recorded behind its last copy has passed.
        self._hosts: list[torch.Tensor | None] = [None, None]
        self._events: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0
        self.last_h2d_bytes = 0
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

    # ------------------------------------------------------------------ fixed-shape decode batches
    @staticmethod
    def decode_layout(padded: int, width: int, n_paged: int) -> tuple[dict[str, tuple[int, int]], int]:
        """Offsets of the sections of a decode batch padded to ``padded`` rows with block tables
        ``width`` wide: the same for every step of that shape, so a captured graph can hold them."""
        off, out = 0, {}
        for name, n in [("tokens", padded), ("positions", padded), ("seq_of_token", padded), ("cu_q", padded + 1),
                        ("kv_len", padded), ("logit_rows", padded), ("dec_tokens", padded), ("dec_seqs", padded),
                        *[(f"bt{g}", padded * width) for g in range(n_paged)]]:
            out[name] = (off, n)
            off += _round4(n)
        return out, off

    def build_decode(self, entries: Sequence[StepEntry], starts: Sequence[int], padded: int, width: int,
                     dev: torch.Tensor) -> StepContext:
        """One token for each request, padded to ``padded`` rows (padding rows hold nothing: context
        length 0 and a block table of -1, so they read and write no page), into the buffer ``dev``."""
        m = self.manager
        B = len(entries)
        paged = [(gi, g) for gi, g in enumerate(m.groups) if isinstance(g, PagedGroup)]
        layout, total = self.decode_layout(padded, width, len(paged))
        host, _ = self._buffers(total)
        h = host.numpy()
        ar = np.arange(padded + 1, dtype=np.int32)

        def put(name, values, fill=0):
            o, n = layout[name]
            h[o:o + n] = fill
            h[o:o + len(values)] = values

        put("tokens", [e.tokens[0] for e in entries])
        put("positions", list(starts))
        put("seq_of_token", ar[:padded])
        put("cu_q", ar)
        put("kv_len", [s + 1 for s in starts])
        put("logit_rows", ar[:padded])
        put("dec_tokens", ar[:padded])
        put("dec_seqs", ar[:padded])
        for k, (gi, g) in enumerate(paged):
            o, n = layout[f"bt{k}"]
            table = h[o:o + n].reshape(padded, width)
            table[:] = -1
            for i, e in enumerate(entries):
                t = g.tables[e.request]
                table[i, :len(t)] = t
        dev[:total].copy_(host[:total], non_blocking=True)
        self.last_h2d_bytes = total * 4
        if self.device.type == "cuda":
            if self._events[self._turn] is None:
                self._events[self._turn] = torch.cuda.Event()
            self._events[self._turn].record()
        view = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
        kv_lens = [s + 1 for s in starts]
        ctx = StepContext(
            num_tokens=padded, num_seqs=padded, num_logit_rows=padded, tokens=view("tokens"),
            positions=view("positions"), seq_of_token=view("seq_of_token"), cu_q=view("cu_q"), kv_len=view("kv_len"),
            logit_rows=view("logit_rows"), requests=[e.request for e in entries], q_lens=[1] * padded,
            kv_lens=kv_lens + [0] * (padded - B))
        for k, (gi, g) in enumerate(paged):
            ctx.block_tables[gi] = view(f"bt{k}").view(padded, width)
        ctx.work = {"dec_tokens": view("dec_tokens"), "dec_seqs": view("dec_seqs"), "n_dec": padded, "n_tiles": 0,
                    "tile_seq": view("dec_seqs")[:0], "tile_q0": view("dec_seqs")[:0],
                    "max_dec_kv": width * m.page_size}
        return ctx

    def build(self, entries: Sequence[StepEntry], starts: Sequence[int], extra_sections: dict[str, np.ndarray] | None = None) -> StepContext:
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
            ("kv_len", np.asarray(kv_lens, dtype=np.int32)), ("logit_rows", np.asarray(rows, dtype=np.int32))]
        shapes: dict[str, tuple] = {}
        for gi, g in enumerate(m.groups):
            if isinstance(g, PagedGroup):
                W = max(1, max((g.pages_for(k) for k in kv_lens), default=1))
                table = np.full((B, W), -1, dtype=np.int32)
                for i, e in enumerate(entries):
                    t = g.tables[e.request]
                    n = min(len(t), W)
                    table[i, :n] = t[:n]
                sections.append((f"bt{gi}", table.reshape(-1)))
                shapes[f"bt{gi}"] = (B, W)
            else:
                sections.append((f"st{gi}", np.asarray([g.slot_of[e.request] for e in entries], dtype=np.int32)))
        # work lists of the attention kernels: requests with one token (decoding) and tiles of
        # QUERY_TILE tokens of the requests with more (portions of prompts)
        ql = np.asarray(q_lens, dtype=np.int32)
        dec = np.nonzero(ql == 1)[0].astype(np.int32)
        tile_seq, tile_q0 = [], []
        for i in np.nonzero(ql > 1)[0]:
            starts_i = np.arange(0, q_lens[i], QUERY_TILE, dtype=np.int32)[::-1]   # late tiles see most keys: first
            tile_seq.append(np.full(starts_i.size, i, dtype=np.int32))
            tile_q0.append(starts_i)
        work_counts = {"dec": int(dec.size), "tiles": int(sum(t.size for t in tile_seq))}
        sections += [("dec_tokens", cu[:-1][dec]), ("dec_seqs", dec),
                     ("tile_seq", np.concatenate(tile_seq) if tile_seq else np.zeros(0, np.int32)),
                     ("tile_q0", np.concatenate(tile_q0) if tile_q0 else np.zeros(0, np.int32))]
        for name, arr in (extra_sections or {}).items():
            sections.append((name, np.ascontiguousarray(arr, dtype=np.int32).reshape(-1)))

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
        if self.device.type == "cuda":
            if self._events[self._turn] is None:
                self._events[self._turn] = torch.cuda.Event()
            self._events[self._turn].record()

        def view(name: str) -> torch.Tensor:
            o, n = offsets[name]
            return dev[o:o + n]

        ctx = StepContext(
            num_tokens=T, num_seqs=B, num_logit_rows=R, tokens=view("tokens"), positions=view("positions"),
            seq_of_token=view("seq_of_token"), cu_q=view("cu_q"), kv_len=view("kv_len"), logit_rows=view("logit_rows"),
            requests=[e.request for e in entries], q_lens=q_lens, kv_lens=kv_lens)
        for gi, g in enumerate(m.groups):
            if isinstance(g, PagedGroup):
                ctx.block_tables[gi] = view(f"bt{gi}").view(shapes[f"bt{gi}"])
            else:
                ctx.state_slots[gi] = view(f"st{gi}")
        for name in ("dec_tokens", "dec_seqs", "tile_seq", "tile_q0", *(extra_sections or {})):
            ctx.work[name] = view(name)
        ctx.work["n_dec"] = work_counts["dec"]
        ctx.work["n_tiles"] = work_counts["tiles"]
        ctx.work["max_dec_kv"] = max((k for k, q in zip(kv_lens, q_lens) if q == 1), default=0)
        return ctx
