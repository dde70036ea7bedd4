"""y = x @ W^T, W stored [out, in]; no bias.

float32 runs: the product is the CUDA-core kernel with true 32-bit accumulation.
bfloat16 runs: the reference hands every bf16 dense product to cuBLAS through
``F.linear`` (acvram/kernels/__init__.py:1896-1899); so may this engine, and it
does for the shapes its own tensor-core kernel does not take.  Logits are the
exception in both: bfloat16 operands, accumulated and returned in float32
(acvram/engine/model.py:369-410), by a kernel of this package.
"""

from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor) -> None:
        self.weight = weight.contiguous()
        self.out_features, self.in_features = self.weight.shape

    @classmethod
    def stacked(cls, weights: list[torch.Tensor]) -> "Linear":
        """One product for several projections of the same input: rows concatenated
        (the reference stacks q,k,v and gate,up at load, acvram/engine/layers.py:1476-1560)."""
        return cls(torch.cat(list(weights), dim=0))

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        w = self.weight
        out_dtype = out_dtype or x.dtype
        out = torch.empty((x.shape[0], self.out_features), device=x.device, dtype=out_dtype)
        if x.shape[0] == 0:
            return out
        if x.dtype == torch.float32:
            return ops.gemm_simt(x, w, out)
        if out_dtype == torch.float32:
            return ops.linear_bf16_f32out(x, w, out, static_weights=True)
        return ops.linear_bf16(x, w, out, static_weights=True)
