"""Sampling parameters, with the reference's names, defaults and meanings
(acvram/engine/sampler.py:20-45)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0          # <= 0: greedy
    top_p: float = 1.0
    top_k: int = 0                    # 0: off
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    max_tokens: int = 512
    stop: list[str] = field(default_factory=list)          # strings that end the request; need the engine's tokenizer
    stop_token_ids: list[int] = field(default_factory=list)
    seed: Optional[int] = None        # the reference stores it and never uses it; here it keys the request's generator
    n: int = 1
    logprobs: Optional[int] = None
    ignore_eos: bool = False          # go on past EOS up to max_tokens; stop_token_ids still stop

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @property
    def penalised(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
