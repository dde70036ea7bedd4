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


class Sampler:
    def __init__(self, device) -> None:
        self.device = torch.device(device)

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
        if penalised:
            logits = logits.clone()
            rows, toks, counts = [], [], []
            for i in penalised:
                c = Counter(histories[i])
                rows += [i] * len(c)
                toks += list(c.keys())
                counts += list(c.values())
            packed = torch.tensor([rows, toks, counts], dtype=torch.int32).to(self.device, non_blocking=True)
            fl = torch.tensor([[p.repetition_penalty for p in params], [p.presence_penalty for p in params],
                               [p.frequency_penalty for p in params]], dtype=torch.float32).to(self.device)
            ops.apply_penalties(logits, packed[0], packed[1], packed[2], fl[0], fl[1], fl[2])
        fl = torch.tensor([[p.temperature for p in params], [p.top_p for p in params], [p.min_p for p in params]],
                          dtype=torch.float32).to(self.device, non_blocking=True)
        top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32).to(self.device, non_blocking=True)
        sc = torch.from_numpy(np.asarray([[s & 0x7FFFFFFFFFFFFFFF for s in seeds], list(counters)],
                                         dtype=np.int64)).to(self.device, non_blocking=True)
        logprobs = torch.empty(R, device=self.device, dtype=torch.float32) if want_logprobs else None
        ops.sample(logits, fl[0], top_k, fl[1], fl[2], sc[0], sc[1], tokens, logprobs)
        return tokens, logprobs
