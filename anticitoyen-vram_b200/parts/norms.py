"""RMS norm with the residual sum fused in."""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import Norm, Runtime
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """out = cast(x32 * rsqrt(mean(x32^2) + eps)) * w, the weight being plain ``w``
    (acvram/engine/layers.py:607-630); with ``delta`` the sum x + delta is made first,
    in 32-bit, and written back (acvram/engine/layers.py:633-651)."""

    def __init__(self, hidden_size: int, eps: float, size: int | None = None) -> None:
        self.size = size or hidden_size
        self.eps = float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.size,), "norm")}

    def load(self, tensors, rt: Runtime) -> None:
        self.weight = tensors["weight"].to(device=rt.device, dtype=torch.float32).contiguous()

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this norm."""
        return {"weight": self.weight, "eps": self.eps}

    def weight_bytes(self) -> int:
        return 0 if self.weight is None else self.weight.numel() * 4

    def forward(self, x, delta, rows=None):
        n = rows.shape[0] if rows is not None else x.shape[0]
        out = torch.empty((n, x.shape[1]), device=x.device, dtype=x.dtype)
        return ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
