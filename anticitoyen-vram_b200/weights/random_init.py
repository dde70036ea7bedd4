"""Random weights from a configuration and a seed.

Matrices and the embedding are N(0, 0.02); every norm weight is 1 + N(0, 0.1),
"random around 1 so that a test that ignored them would not stay close"
(the reference's own test fixtures do so for q_norm/k_norm,
tests/conftest.py:141-183).  Each tensor has its own generator, seeded by
(seed, tensor name), so a tensor's values do not depend on which others are made
nor on their order.  Values are rounded to bfloat16, so that a folder written
here reads the same in both run precisions.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator, Mapping

import torch
from safetensors.torch import save_file

from .needs import TensorNeed


def _seed_of(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, need: TensorNeed, seed: int, device: str | torch.device = "cpu",
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_of(seed, name))
    if need.role == "table":
        return torch.randint(0, 2 ** 15, need.shape, generator=gen, device=device, dtype=torch.int32)
    noise = torch.empty(need.shape, device=device, dtype=torch.float32).normal_(0.0, 1.0, generator=gen)
    if need.role == "norm":
        noise.mul_(0.1).add_(1.0)
    else:
        noise.mul_(0.02)
    return noise.to(dtype)


def random_tensors(needs: Mapping[str, TensorNeed], seed: int, device: str | torch.device = "cpu",
                   dtype: torch.dtype = torch.bfloat16) -> Iterator[tuple[str, torch.Tensor]]:
    for name, need in needs.items():
        if need.optional:
            continue
        yield name, random_tensor(name, need, seed, device, dtype)


def write_random_model(config, folder: str | os.PathLike, seed: int = 0,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` into ``folder``.

    ``config`` is a typed configuration of a registered architecture.  ``dtype``
    is the stored type; float32 files hold the same bfloat16-rounded values."""
    from ..config import family_of
    from ..models import needs_of_plan

    folder = os.fspath(folder)
    os.makedirs(folder, exist_ok=True)
    cfg = config.to_dict()
    plan = family_of(cfg).build_plan(config)
    tensors = {name: t.to(dtype).contiguous()
               for name, t in random_tensors(needs_of_plan(plan), seed, "cpu", torch.bfloat16)}
    cfg["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
