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

from dataclasses import dataclass, field
from typing import Mapping

import torch

from ..weights.needs import TensorNeed


@dataclass
class Runtime:
    """Where and in which precision a model runs."""

    device: torch.device
    dtype: torch.dtype  # torch.float32: everything in true 32-bit; torch.bfloat16: the serving precision


@dataclass
class StepMetadata:
    """What a mixer asks of every step beside the generic batch: int32 ``arrays`` that travel to the device with
    the step's tokens, and plain ``values`` (counts, maxima) that stay on the host.  Both arrive as one dict in
    ``StepContext.work[key]``, the arrays as views of the step's device buffer."""

    arrays: Mapping = field(default_factory=dict)
    values: Mapping = field(default_factory=dict)


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
    capturable = True     # forward only launches kernels (no read of device memory by the host): may run in a CUDA graph

    def tensor_needs(self) -> Mapping[str, TensorNeed]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        pass

    # ---- what a step costs, for measurement (a roofline follows the plan, not an architecture's formula)
    def weight_bytes(self) -> int:
        """Bytes of weights that one step reads (each once, whatever the batch)."""
        return 0

    def flops(self, num_tokens: int) -> float:
        """Floating-point operations of the part's matrix products for ``num_tokens`` tokens."""
        return 0.0


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
    # A mixer whose kernels need per-step data of their own (work lists, tiles) names a key here and offers
    # ``step_metadata(q_lens, kv_lens, cu_q) -> StepMetadata`` for any batch and ``decode_metadata(padded, max_kv)``
    # for a batch of ``padded`` one-token requests with contexts up to ``max_kv`` (arrays of fixed size: they are
    # written once into a captured graph's buffer).  Mixers with the same key share one set per step.
    metadata_key: str | None = None

    def cache_need(self):
        """PagedNeed, StateNeed or None: what this mixer keeps for each request."""
        return None

    def mixing_flops(self, q_lens, kv_lens) -> float:
        """Operations of the mixing itself (scores and weighted sums) for requests that bring ``q_lens`` tokens
        and hold ``kv_lens`` after the step."""
        return 0.0

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        """Bytes of cache that the step has to read for these requests."""
        return 0

    def forward(self, h: torch.Tensor, ctx, cache: CacheView | None) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError
