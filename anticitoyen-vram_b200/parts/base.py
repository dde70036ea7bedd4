"""Interfaces of the parts.

Every part
  * is built from sizes and constants only (``hidden_size`` plus its PartSpec's
    parameters) and never learns which model it is in;
  * names the tensors it reads, relative to its layer's prefix
    (``tensor_needs``), and takes them in ``load``;
  * runs on the tokens of one step, given as a ``StepContext``
    (acvram_b200.engine.batch), with hand-written kernels only.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping

import torch

from ..weights.needs import TensorNeed


@dataclass
class Runtime:
    """Where and in which precision a model runs."""

    device: torch.device
    dtype: torch.dtype  # torch.float32: everything in true 32-bit; torch.bfloat16: the serving precision


@dataclass
class CacheView:
    """What a mixer gets of the cache for one run of its layer."""

    group: int                      # index of the cache group (for the step's block table or state slots)
    writes: bool                    # False: read what another layer wrote
    k_pages: torch.Tensor | None = None
    v_pages: torch.Tensor | None = None
    state: torch.Tensor | None = None   # [max_requests, *shape] for a StateNeed


class Part:
    kind = "?"

    def tensor_needs(self) -> Mapping[str, TensorNeed]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        pass


class Norm(Part):
    def forward(self, x: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor | None = None) -> torch.Tensor:
        """x += delta in place (if given), return norm(x); with ``rows`` only those rows, x untouched."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Either gives a rotary table that the attention kernel applies itself
    (``rotary_table``), or changes q and k in place between norm and append (``apply``)."""

    def rotary_table(self) -> torch.Tensor | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        """q: [T, NH, D] view, k: [T, NKV, D] view, both changed in place."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        """PagedNeed, StateNeed or None: what this mixer keeps for each request."""
        return None

    def forward(self, h: torch.Tensor, ctx, cache: CacheView | None) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError
