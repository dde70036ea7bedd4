"""y = x @ W^T (+ b), W stored [out, in].

float32 runs: the product is the CUDA-core kernel with true 32-bit accumulation.
bfloat16 runs: the reference hands every bf16 dense product to cuBLAS through
``F.linear`` (acvram/kernels/__init__.py:1896-1899); so may this engine, and it
does for the shapes its own tensor-core kernel does not take.  Logits are the
exception in both: bfloat16 operands, accumulated and returned in float32
(acvram/engine/model.py:369-410), by a kernel of this package.

A bias is there when the weight file holds one, as in the reference
(acvram/engine/loader.py:269-270); it is kept in float32 and added by a kernel of
its own after the product.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.needs import TensorNeed


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        self.weight = weight.contiguous()
        self.out_features, self.in_features = self.weight.shape
        self.bias = None if bias is None else bias.to(device=weight.device, dtype=torch.float32).contiguous()

    @classmethod
    def stacked(cls, weights: list[torch.Tensor], biases: list | None = None) -> "Linear":
        """One product for several projections of the same input: rows concatenated
        (the reference stacks q,k,v and gate,up at load, acvram/engine/layers.py:1476-1560).
        ``biases``: one per projection or None; where some have one and others not, the others get zeros."""
        bias = None
        if biases is not None and any(b is not None for b in biases):
            bias = torch.cat([b.float() if b is not None else torch.zeros(w.shape[0], device=w.device)
                              for w, b in zip(weights, biases)])
        return cls(torch.cat(list(weights), dim=0), bias)

    @staticmethod
    def needs(prefix: str, out_features: int, in_features: int, bias: bool | None) -> dict[str, TensorNeed]:
        """``prefix + "weight"`` and, with ``bias`` True, ``prefix + "bias"``; None: the bias is read if the file has it."""
        needs = {prefix + "weight": TensorNeed((out_features, in_features))}
        if bias is not False:
            needs[prefix + "bias"] = TensorNeed((out_features,), "bias", optional=bias is None)
        return needs

    def weight_bytes(self) -> int:
        n = self.weight.numel() * self.weight.element_size()
        return n + (self.bias.numel() * 4 if self.bias is not None else 0)

    def flops(self, tokens: int) -> float:
        return 2.0 * tokens * self.out_features * self.in_features

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        out_dtype = out_dtype or x.dtype
        out = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=out_dtype)
        if x.shape[0] == 0:
            return out
        if x.dtype == torch.float32:
            ops.gemm_simt(x, w, out)
        elif out_dtype == torch.float32:
            ops.linear_bf16_f32out(x, w, out, static_weights=True)
        else:
            ops.linear_bf16(x, w, out, static_weights=True)
        if self.bias is not None:
            ops.add_bias(out, self.bias)
        return out
