"""The step function: run a batch of (request, its next tokens) from the cache.

``ModelRunner`` owns the model, the cache manager and the cache storage.  One
call of ``step`` reserves pages for the tokens it is given, runs exactly those
tokens as one batch through every scheduled layer (reading older keys and values
from the pages that earlier steps left), and returns float32 logits at the wanted
places.  Generation (the scheduler) and trace replay both go through this call.
"""

from __future__ import annotations

from typing import Hashable, Sequence

import torch

from ..cache import CacheManager, CacheStorage
from ..kernels import ops
from ..parts import Runtime
from .batch import BatchBuilder, StepContext, StepEntry


class ModelRunner:
    def __init__(self, model, page_size: int, num_pages: int, max_requests: int,
                 enable_prefix_cache: bool = False, max_len: int | None = None) -> None:
        """``max_len``: the longest request in tokens (default: what the model's positions and the pool allow);
        the block tables on the device get that many columns' worth of pages."""
        if model.rt is None:
            raise ValueError("the model has no weights loaded")
        rt: Runtime = model.rt
        self.model = model
        self.rt = rt
        self.manager = CacheManager(model.cache_plan(), page_size, num_pages, max_requests, enable_prefix_cache)
        self.storage = CacheStorage(self.manager, rt.device, rt.dtype, min(max_len or model.plan.max_positions,
                                                                            model.plan.max_positions))
        self.max_len = min(model.plan.max_positions, self.storage.max_tokens)
        self.builder = BatchBuilder(self.manager, self.storage, rt.device, model.plan.vocab_size, self.max_len,
                                    model.metadata_providers() if hasattr(model, "metadata_providers") else {})
        self.steps = 0
        self.graphs = None          # DecodeGraphs when graph replay of decode steps is on

    def enable_graphs(self) -> None:
        """Replay decode steps (one token per request) from captured CUDA graphs."""
        from .graphs import DecodeGraphs
        if self.rt.device.type == "cuda":
            self.graphs = DecodeGraphs(self)

    @property
    def graph_launches(self) -> int:
        return self.graphs.launches if self.graphs is not None else 0

    def check_status(self) -> None:
        """Wait for the device and raise if a kernel gave up one of its bounded waits since the last check: the
        logits of such a step are not to be used.  (``Engine`` reads the same word with every step's tokens.)"""
        if self.rt.device.type != "cuda":
            return
        code = int(ops.status_word(self.rt.device).item())
        if code:
            ops.reset_after_failure()
            raise ops.KernelError(f"a kernel gave up a bounded wait (status {code}); the step's results are not used")

    # ------------------------------------------------------------------ requests
    def admit(self, request: Hashable) -> None:
        self.manager.admit(request)

    def release(self, request: Hashable) -> None:
        self.manager.release(request)

    def length(self, request: Hashable) -> int:
        return self.manager.lengths[request]

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: Sequence[StepEntry]) -> StepContext:
        """Admit new requests, reserve pages for the step's tokens, build its context."""
        m = self.manager
        self.builder.validate(entries)
        for e in entries:
            have = m.lengths.get(e.request, 0)
            if have + len(e.tokens) > self.max_len:
                raise ValueError(f"request {e.request!r} would reach {have + len(e.tokens)} tokens; the model's positions "
                                 f"and the cache hold {self.max_len}")
        starts = []
        for e in entries:
            if e.request not in m.lengths:
                self.admit(e.request)
            start = m.lengths[e.request]
            if start == 0:     # a request's first step (also after a preemption): its state starts at zero
                self._zero_state(e.request)
            m.grow(e.request, start + len(e.tokens))   # takes nothing if the scheduler reserved already
            starts.append(start)
        return self.builder.build(entries, starts)

    def _zero_state(self, request: Hashable) -> None:
        for gi, g in enumerate(self.manager.groups):
            if g.need.kind == "state":
                self.storage.zero_state(gi, g.slot_of[request])

    def _graph_step(self, entries, device_tokens):
        m = self.manager
        self.builder.validate(entries)
        starts = []
        for e in entries:
            if e.request not in m.lengths:
                self.admit(e.request)
            start = m.lengths[e.request]
            if start + 1 > self.max_len:
                raise ValueError(f"request {e.request!r} would pass the {self.max_len} tokens that the model's positions "
                                 f"and the cache hold")
            if start == 0:
                self._zero_state(e.request)
            m.grow(e.request, start + 1)
            starts.append(start)
        with torch.cuda.device(self.rt.device):
            logits = self.graphs.run(entries, starts, device_tokens)
        if logits is None:
            return None
        if any(e.want != (0,) and list(e.want) != [0] for e in entries):
            rows = [i for i, e in enumerate(entries) if len(e.want)]
            logits = logits[rows] if len(rows) != len(entries) else logits
        for e, s in zip(entries, starts):
            m.advance(e.request, s + 1)
            m.trim(e.request)
        self.steps += 1
        return logits

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Logits float32 [wanted, vocab] in the order of the entries and of their ``want``.

        ``device_tokens`` (int32 [T] on the device) replaces the entries' token ids, for a caller that
        keeps the sampled tokens on the device between steps; the entries then only say how many."""
        if not entries:
            return torch.empty((0, self.model.plan.vocab_size), device=self.rt.device, dtype=torch.float32)
        if self.graphs is not None and self.graphs.usable(entries):
            logits = self._graph_step(entries, device_tokens)
            if logits is not None:
                return logits
        ctx = self.prepare(entries)
        if device_tokens is not None:
            ctx.tokens.copy_(device_tokens)
        if self.rt.device.type == "cuda":
            with torch.cuda.device(self.rt.device):
                logits = self.model.forward(ctx, self.storage)
        else:  # only reachable with the kernels replaced by a test: the kernels themselves refuse CPU tensors
            logits = self.model.forward(ctx, self.storage)
        for e, kv in zip(entries, ctx.kv_lens):
            self.manager.advance(e.request, kv)
            self.manager.trim(e.request)
        self.steps += 1
        return logits
