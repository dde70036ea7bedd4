"""Position encodings."""

from __future__ import annotations

import weakref

import torch

from .base import PositionEncoding, Runtime
from .registry import register


@register("position", "rotary")
class Rotary(PositionEncoding):
    """Rotate-half rotary positions over the first ``dim`` elements of a head.

    inv_freq[i] = 1 / theta^(2i/dim); angle = position * inv_freq; pairs are
    (i, i + dim/2) (acvram/engine/layers.py:727-730, 934-936, 1006-1009).  The table
    holds, for each position, cos of the dim/2 angles and then their sin, in
    float32: the reference rounds its tables to the model's type
    (acvram/engine/layers.py:829-830); here angles, cos and sin stay 32-bit in both
    precisions.  The attention kernel reads the table itself.

    Layers with the same (dim, theta, positions) on the same device hold one table between them (the table
    of a model with 40 960 positions and heads of 128 is 21 MB; a copy for each of 36 layers would be 755 MB)."""

    _shared: "weakref.WeakValueDictionary" = weakref.WeakValueDictionary()

    def __init__(self, hidden_size: int, dim: int, theta: float, max_positions: int) -> None:
        if dim % 2:
            raise ValueError(f"rotary dim {dim} must be even")
        self.dim, self.theta, self.max_positions = int(dim), float(theta), int(max_positions)
        self.table: torch.Tensor | None = None

    def load(self, tensors, rt: Runtime) -> None:
        key = (self.dim, self.theta, self.max_positions, str(rt.device))
        table = Rotary._shared.get(key)
        if table is None:
            inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim))
            ang = torch.outer(torch.arange(self.max_positions, dtype=torch.float32), inv)
            table = torch.cat((ang.cos(), ang.sin()), dim=-1).contiguous().to(rt.device)
            Rotary._shared[key] = table
        self.table = table

    def rotary_table(self):
        return self.table


@register("position", "none")
class NoPosition(PositionEncoding):
    """No position signal (the mixer sees order through causality only)."""

    def __init__(self, hidden_size: int) -> None:
        pass

    def apply(self, q, k, ctx) -> None:
        return None
