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

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp.", bias: bool | None = None) -> None:
        """``bias``: True, the three projections have biases; False, none; None, those that the file holds."""
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.prefix = prefix
        self.bias = bias

    def tensor_needs(self):
        H, I = self.hidden_size, self.intermediate_size
        needs = {}
        for name, n_out, n_in in (("gate_proj.", I, H), ("up_proj.", I, H), ("down_proj.", H, I)):
            needs.update(Linear.needs(self.prefix + name, n_out, n_in, self.bias))
        return needs

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def flops(self, num_tokens: int) -> float:
        return self.gate_up.flops(num_tokens) + self.down.flops(num_tokens)

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda n: tensors[n].to(device=rt.device, dtype=rt.dtype)
        b = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32) if n in tensors else None
        gate, up = w(self.prefix + "gate_proj.weight"), w(self.prefix + "up_proj.weight")
        gate_b, up_b, down_b = (b(self.prefix + n) for n in ("gate_proj.bias", "up_proj.bias", "down_proj.bias"))
        # bfloat16 with 16-byte aligned rows: gate and up rows are interleaved (g0, u0, g1, u1 ...) so that the
        # tensor-core product's epilogue holds each pair together and applies SiLU(gate) * up itself; the
        # stacked product's output [T, 2I] is then never written.  Otherwise: stacked product, then the kernel.
        # (with a bias on gate or up the pair goes the unfused way: the epilogue adds none)
        self.fused = rt.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and gate_b is None and up_b is None
        if self.fused:
            self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size))
        else:
            self.gate_up = Linear.stacked([gate, up], [gate_b, up_b])
        self.down = Linear(w(self.prefix + "down_proj.weight"), down_b)

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this feed-forward: gate and up rows interleaved, no biases."""
        if not self.fused or self.down.bias is not None:
            return None
        return {"intermediate_size": self.intermediate_size, "w_gate_up_pairs": self.gate_up.weight, "w_down": self.down.weight}

    def forward(self, h, ctx):
        if self.fused and h.shape[0] and ops.gemm_tc_takes(h, self.gate_up.weight):
            act = torch.empty((h.shape[0], self.intermediate_size), device=h.device, dtype=h.dtype)
            ops.linear_bf16_swiglu(h, self.gate_up.weight, act, static_weights=True)
            return self.down(act)
        if self.fused:      # an input the tensor-core kernel does not take: undo the interleaving for this call
            gu = self.gate_up(h).view(h.shape[0], self.intermediate_size, 2).transpose(1, 2).reshape(h.shape[0], -1)
        else:
            gu = self.gate_up(h)
        act = torch.empty((h.shape[0], self.intermediate_size), device=h.device, dtype=h.dtype)
        ops.swiglu(gu, act)
        return self.down(act)
