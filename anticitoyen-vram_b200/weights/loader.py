"""Read a model folder's safetensors by tensor name.

The folder holds ``model.safetensors``, or ``model.safetensors.index.json`` with
its shards (the reference accepts both at conversion time,
acvram/quant/convert.py:1203-1217, and keeps the tensor names of the file,
acvram/engine/loader.py:403-406, 1013-1033).  The reference reports a missing
name with a KeyError at first use and never checks shapes
(acvram/engine/loader.py:506-508); here the whole file is checked against the
model's needs first and one error lists everything that is missing, unexpected
or of the wrong shape.  Tensors that the model does not use are no fault by
themselves (the reference ignores them): alone they are listed once in a warning
and skipped, unless ``strict`` asks for the error; beside another fault they are
listed in the error with it.

Storage rule: bfloat16 stays bfloat16, float32 stays float32, integer tables
become int32.  float16 becomes float32, which holds every float16 value exactly
(bfloat16 would drop three bits of its mantissa): a float32 run then computes
with the file's own values, and a bfloat16 run rounds them once, where the parts
cast what they compute with.
"""

from __future__ import annotations

import json
import os
import warnings
from typing import Mapping

import torch
from safetensors import safe_open

from .needs import TensorNeed, WeightError

_KEEP = {torch.bfloat16: torch.bfloat16, torch.float16: torch.float32, torch.float32: torch.float32,
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


class UnusedTensorsWarning(UserWarning):
    """The weight file holds tensors that the model does not read."""


def load_tensors(folder: str | os.PathLike, needs: Mapping[str, TensorNeed],
                 device: str | torch.device = "cpu", strict: bool = False) -> dict[str, torch.Tensor]:
    """Return ``{name: tensor}`` for every needed tensor that the folder holds.

    ``strict``: tensors that the model does not use are an error even when nothing else is wrong."""
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
        if missing or wrong_shape or (unexpected and strict):
            raise WeightError(folder, missing, unexpected, wrong_shape)
        if unexpected:
            shown = ", ".join(unexpected[:8]) + (f" and {len(unexpected) - 8} more" if len(unexpected) > 8 else "")
            warnings.warn(f"weights in {folder}: {len(unexpected)} tensors that the model does not use are skipped: {shown}",
                          UnusedTensorsWarning, stacklevel=2)
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
