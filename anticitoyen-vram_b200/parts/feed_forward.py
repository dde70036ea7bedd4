"""Feed-forward parts."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import FeedForward, Runtime
from .linear import Linear
from .registry import register


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """y = (silu(x Wg^T) * (x Wu^T)) Wd^T, gate and up as one stacked product
    (acvram/engine/attention.py:705-783)."""

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp.") -> None:
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.prefix = prefix

    def tensor_needs(self):
        H, I = self.hidden_size, self.intermediate_size
        return {self.prefix + "gate_proj.weight": TensorNeed((I, H)), self.prefix + "up_proj.weight": TensorNeed((I, H)),
                self.prefix + "down_proj.weight": TensorNeed((H, I))}

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda n: tensors[n].to(device=rt.device, dtype=rt.dtype)
        self.gate_up = Linear.stacked([w(self.prefix + "gate_proj.weight"), w(self.prefix + "up_proj.weight")])
        self.down = Linear(w(self.prefix + "down_proj.weight"))

    def forward(self, h, ctx):
        gu = self.gate_up(h)
        act = torch.empty((h.shape[0], self.intermediate_size), device=h.device, dtype=h.dtype)
        ops.swiglu(gu, act)
        return self.down(act)
