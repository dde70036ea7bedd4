"""Read a model folder's safetensors by tensor name.

The folder holds ``model.safetensors``, or ``model.safetensors.index.json`` with
its shards (the reference accepts both at conversion time,
acvram/quant/convert.py:1203-1217, and keeps the tensor names of the file,
acvram/engine/loader.py:403-406, 1013-1033).  The reference reports a missing
name with a KeyError at first use and never checks shapes
(acvram/engine/loader.py:506-508); here the whole file is checked against the
model's needs first and one error lists everything that is missing, unexpected
or of the wrong shape.

Storage rule: floating tensors stored in 16 bits are kept as bfloat16, tensors
stored in 32-bit floating point stay float32, integer tables become int32.  The
parts cast what they compute with.
"""

from __future__ import annotations

import json
import os
from typing import Mapping

import torch
from safetensors import safe_open

from .needs import TensorNeed, WeightError

_KEEP = {torch.bfloat16: torch.bfloat16, torch.float16: torch.bfloat16, torch.float32: torch.float32,
         torch.int32: torch.int32, torch.int64: torch.int32, torch.int16: torch.int32, torch.int8: torch.int32,
         torch.uint8: torch.int32}


def _files_of(folder: str) -> dict[str, list[str] | None]:
    """file path -> tensor names to take from it (None: all of them)."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(single):
        return {single: None}
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            weight_map = json.load(fh).get("weight_map", {})
        files: dict[str, list[str]] = {}
        for name, shard in weight_map.items():
            files.setdefault(os.path.join(folder, shard), []).append(name)
        return files
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {folder}")


def load_tensors(folder: str | os.PathLike, needs: Mapping[str, TensorNeed],
                 device: str | torch.device = "cpu") -> dict[str, torch.Tensor]:
    """Return ``{name: tensor}`` for every needed tensor that the folder holds."""
    folder = os.fspath(folder)
    files = _files_of(folder)
    present: dict[str, tuple[str, tuple[int, ...]]] = {}
    handles = {}
    try:
        for path, names in files.items():
            if not os.path.isfile(path):
                raise FileNotFoundError(f"shard {path} named by the index is absent")
            fh = safe_open(path, framework="pt", device="cpu")
            handles[path] = fh
            for name in (fh.keys() if names is None else names):
                present[name] = (path, tuple(fh.get_slice(name).get_shape()))
        missing = [n for n, need in needs.items() if n not in present and not need.optional]
        unexpected = sorted(n for n in present if n not in needs)
        wrong_shape = [(n, present[n][1], need.shape) for n, need in needs.items()
                       if n in present and present[n][1] != tuple(need.shape)]
        if missing or unexpected or wrong_shape:
            raise WeightError(folder, missing, unexpected, wrong_shape)
        out: dict[str, torch.Tensor] = {}
        wrong_dtype = []
        for name in needs:
            if name not in present:
                continue
            tensor = handles[present[name][0]].get_tensor(name)
            keep = _KEEP.get(tensor.dtype)
            if keep is None:
                wrong_dtype.append((name, str(tensor.dtype)))
                continue
            out[name] = tensor.to(device=device, dtype=keep)
        if wrong_dtype:
            raise WeightError(folder, wrong_dtype=wrong_dtype)
        return out
    finally:
        handles.clear()
