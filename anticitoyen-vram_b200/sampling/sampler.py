"""Choose the next token of each row of a logits batch, on the device.

Order as in the reference (acvram/engine/sampler.py:195-256): penalties on the raw
logits, temperature, top-k, min-p, top-p, draw; a batch that is all greedy and
unpenalised is one argmax.  The history of a request is consulted only when its
row is penalised (acvram/engine/sampler.py:73-84 builds it only off the greedy
path for the same reason).  Each row draws from its own counter-based generator
(seed of the request, index of the token being drawn), so a request's tokens do
not depend on what else is in the batch.
"""

from __future__ import annotations

from collections import Counter
from typing import Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


def _round4(n: int) -> int:
    return (n + 3) & ~3


class Sampler:
    """The per-row parameters of a step (temperature, top-p, min-p, top-k, seed, counter) travel to the device in
    one copy from pinned memory: two staging buffers in turn, each rewritten only after its last copy has gone."""

    def __init__(self, device) -> None:
        self.device = torch.device(device)
        self._hosts: list[torch.Tensor | None] = [None, None]
        self._events: list = [None, None]
        self._devs: list[torch.Tensor | None] = [None, None]
        self._turn = 0

    def _stage(self, ints: int) -> tuple[torch.Tensor, torch.Tensor]:
        self._turn ^= 1
        i = self._turn
        if self._events[i] is not None:
            self._events[i].synchronize()
        if self._hosts[i] is None or self._hosts[i].numel() < ints:
            cap = max(1024, 1 << (ints - 1).bit_length())
            self._hosts[i] = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
            self._devs[i] = torch.empty(cap, dtype=torch.int32, device=self.device)
        return self._hosts[i], self._devs[i]

    def _send(self, host: torch.Tensor, dev: torch.Tensor, ints: int) -> None:
        dev[:ints].copy_(host[:ints], non_blocking=True)
        if self.device.type == "cuda":
            if self._events[self._turn] is None:
                self._events[self._turn] = torch.cuda.Event()
            self._events[self._turn].record()

    def __call__(self, logits: torch.Tensor, params: Sequence[SamplingParams], histories: Sequence[Sequence[int]],
                 seeds: Sequence[int], counters: Sequence[int], want_logprobs: bool = False):
        """logits float32 [R, V] -> (tokens int32 [R] on the device, logprobs float32 [R] or None)."""
        R = logits.shape[0]
        tokens = torch.empty(R, device=self.device, dtype=torch.int32)
        if R == 0:
            return tokens, None
        penalised = [i for i, p in enumerate(params) if p.penalised and histories[i]]
        if not penalised and all(p.greedy for p in params) and not want_logprobs:
            return ops.argmax(logits, tokens), None
        # one buffer: [temperature | top_p | min_p | repetition | presence | frequency] float32, [top_k] int32,
        # [seed | counter] int64, then (row, token, count) of the penalised rows' histories
        R4 = _round4(R)
        rows, toks, counts = [], [], []
        for i in penalised:
            c = Counter(histories[i])
            rows += [i] * len(c)
            toks += list(c.keys())
            counts += list(c.values())
        n_pen = len(rows)
        o_k, o_seed, o_pen = 6 * R4, 8 * R4, 8 * R4 + 4 * R4
        ints = o_pen + 3 * _round4(n_pen)
        host, dev = self._stage(ints)
        h = host.numpy()
        hf = h.view(np.float32)
        for j, name in enumerate(("temperature", "top_p", "min_p", "repetition_penalty", "presence_penalty",
                                  "frequency_penalty")):
            hf[j * R4:j * R4 + R] = [getattr(p, name) for p in params]
        h[o_k:o_k + R] = [p.top_k for p in params]
        h64 = h[o_seed:o_seed + 4 * R4].view(np.int64)
        h64[:R] = [s & 0x7FFFFFFFFFFFFFFF for s in seeds]
        h64[R4:R4 + R] = list(counters)
        if n_pen:
            P4 = _round4(n_pen)
            h[o_pen:o_pen + n_pen] = rows
            h[o_pen + P4:o_pen + P4 + n_pen] = toks
            h[o_pen + 2 * P4:o_pen + 2 * P4 + n_pen] = counts
        self._send(host, dev, ints)
        f = lambda j: dev[j * R4:j * R4 + R].view(torch.float32)
        d64 = dev[o_seed:o_seed + 4 * R4].view(torch.int64)
        if n_pen:
            P4 = _round4(n_pen)
            logits = logits.clone()
            ops.apply_penalties(logits, dev[o_pen:o_pen + n_pen], dev[o_pen + P4:o_pen + P4 + n_pen],
                                dev[o_pen + 2 * P4:o_pen + 2 * P4 + n_pen], f(3), f(4), f(5))
        logprobs = torch.empty(R, device=self.device, dtype=torch.float32) if want_logprobs else None
        ops.sample(logits, f(0), dev[o_k:o_k + R], f(1), f(2), d64[:R], d64[R4:R4 + R], tokens, logprobs)
        return tokens, logprobs
