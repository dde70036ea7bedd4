"""Random weights from a configuration and a seed.

Matrices and the embedding are N(0, 0.02); every norm weight is 1 + N(0, 0.1),
"random around 1 so that a test that ignored them would not stay close"
(the reference's own test fixtures do so for q_norm/k_norm,
tests/conftest.py:141-183).  Each tensor has its own generator, keyed by
(seed, tensor name), so a tensor's values do not depend on which others are made,
on their order, nor on where they are made: the generator is counter-based
(Philox-4x32-10) and the normal deviates come from tabulated quantiles with
rounded float additions and multiplications only, arithmetic that numpy on the
host and the kernel on the device (csrc/random_fill.cu) carry out bit for bit
alike.  ``Engine(config, random_weights=True, seed=S)``, which draws on the
device, therefore holds the same model as a folder written with the same seed.
Values are rounded to bfloat16, so that a folder written here reads the same in
both run precisions.
"""

from __future__ import annotations

import hashlib
import json
import os
from statistics import NormalDist
from typing import Iterator, Mapping

import numpy as np
import torch
from safetensors.torch import save_file

from .needs import TensorNeed

_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_TABLES: tuple[np.ndarray, np.ndarray] | None = None
_DEVICE_TABLES: dict = {}


def _seed_of(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def quantile_tables() -> tuple[np.ndarray, np.ndarray]:
    """(t1 [1024], t2 [1025]) float32: t1[k] is the k/1024 quantile of the half-normal; t2 cuts the last of
    these intervals into 1024 again, and ends at the quantile of the largest 31-bit fraction."""
    global _TABLES
    if _TABLES is None:
        inv = NormalDist().inv_cdf
        t1 = np.array([inv(0.5 + (k / 1024) / 2) for k in range(1024)], dtype=np.float64)
        t2 = [inv(0.5 + (1023 / 1024 + (k / 1024) / 1024) / 2) for k in range(1024)]
        t2.append(inv(1.0 - 2.0 ** -32))
        _TABLES = (t1.astype(np.float32), np.array(t2, dtype=np.float64).astype(np.float32))
    return _TABLES


def philox_words(seed: int, first_block: int, num_blocks: int) -> np.ndarray:
    """Philox-4x32-10 (Salmon et al., SC'11): uint32 [4 * num_blocks], the four words of counters
    first_block .. first_block + num_blocks - 1 under the 64-bit key ``seed``."""
    ctr = np.arange(first_block, first_block + num_blocks, dtype=np.uint64)
    c0, c1 = ctr & _MASK, ctr >> np.uint64(32)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    s32 = np.uint64(32)
    for _ in range(10):
        p0 = np.uint64(_M0) * c0
        p1 = np.uint64(_M1) * c2
        c0, c1, c2, c3 = (p1 >> s32) ^ c1 ^ np.uint64(k0), p1 & _MASK, (p0 >> s32) ^ c3 ^ np.uint64(k1), p0 & _MASK
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32).reshape(-1)


def normal_of_words(words: np.ndarray) -> np.ndarray:
    """Standard normal deviates (float32) of uint32 words: sign bit, then the inverse CDF of the half-normal,
    piecewise linear between the tabulated quantiles (see csrc/random_fill.cu for the same steps)."""
    t1, t2 = quantile_tables()
    r = words & np.uint32(0x7FFFFFFF)
    i = (r >> np.uint32(21)).astype(np.int64)
    tail = i >= 1023
    j = ((r >> np.uint32(11)) & np.uint32(1023)).astype(np.int64)
    ii = np.minimum(i, 1022)
    a = np.where(tail, t2[j], t1[ii]).astype(np.float32)
    b = np.where(tail, t2[j + 1], t1[ii + 1]).astype(np.float32)
    frac = np.where(tail, (r & np.uint32(0x7FF)).astype(np.float32) * np.float32(2.0 ** -11),
                    (r & np.uint32(0x1FFFFF)).astype(np.float32) * np.float32(2.0 ** -21)).astype(np.float32)
    m = a + (b - a) * frac                      # three float32 operations, each rounded
    return np.where(words >> np.uint32(31), -m, m).astype(np.float32)


def _host_tensor(need: TensorNeed, key: int, dtype: torch.dtype) -> torch.Tensor:
    n = 1
    for d in need.shape:
        n *= d
    chunk = 1 << 20                              # counters per pass: a few tens of MB of temporaries
    if need.role == "table":
        out = np.empty(n, dtype=np.int32)
    else:
        out = np.empty(n, dtype=np.float32)
        mean, std = (1.0, 0.1) if need.role == "norm" else (0.0, 0.02)
    for b0 in range(0, (n + 3) // 4, chunk):
        words = philox_words(key, b0, min(chunk, (n + 3) // 4 - b0))
        lo = 4 * b0
        hi = min(n, lo + words.size)
        if need.role == "table":
            out[lo:hi] = (words[:hi - lo] & np.uint32(0x7FFF)).astype(np.int32)
        else:
            out[lo:hi] = np.float32(mean) + np.float32(std) * normal_of_words(words[:hi - lo])
    t = torch.from_numpy(out).view(need.shape)
    return t if need.role == "table" else t.to(dtype)


def _device_tensor(need: TensorNeed, key: int, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    from ..kernels import ops
    tables = _DEVICE_TABLES.get(str(device))
    if tables is None:
        tables = _DEVICE_TABLES[str(device)] = tuple(torch.from_numpy(t).to(device) for t in quantile_tables())
    if need.role == "table":
        return ops.random_int(torch.empty(need.shape, device=device, dtype=torch.int32), key, 0x7FFF)
    mean, std = (1.0, 0.1) if need.role == "norm" else (0.0, 0.02)
    if dtype not in (torch.float32, torch.bfloat16):
        return ops.random_normal(torch.empty(need.shape, device=device, dtype=torch.float32), key, mean, std, *tables).to(dtype)
    return ops.random_normal(torch.empty(need.shape, device=device, dtype=dtype), key, mean, std, *tables)


def random_tensor(name: str, need: TensorNeed, seed: int, device: str | torch.device = "cpu",
                  dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The tensor that (seed, name) stands for, made where it is wanted: the same bits on the host and on a device."""
    device = torch.device(device)
    key = _seed_of(seed, name)
    if device.type == "cuda":
        return _device_tensor(need, key, device, dtype)
    return _host_tensor(need, key, dtype)


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
    tensors = {name: t.to(dtype).contiguous() if t.is_floating_point() else t.contiguous()
               for name, t in random_tensors(needs_of_plan(plan), seed, "cpu", torch.bfloat16)}
    cfg["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(cfg, fh, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
