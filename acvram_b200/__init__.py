"""acvram_b200 -- a small, whole inference engine for one B200 (sm_100a).

The source tree of the package is the folder ``anticitoyen-vram_b200/`` beside
this one; its name carries a hyphen and cannot be written in an ``import``
statement, so this module is the importable name and lends its ``__path__`` to
that folder.  Every submodule is therefore ``acvram_b200.<subpackage>``
(``acvram_b200.config``, ``acvram_b200.engine`` ...), and is loaded once.

Public entry points (imported lazily, so that ``import acvram_b200`` needs no
GPU and compiles nothing):

    Engine, SamplingParams, GenerationOutput   -- acvram_b200.engine
    load_config, REGISTRY                      -- acvram_b200.config
    write_random_model                         -- acvram_b200.weights
"""

from __future__ import annotations

import importlib
import pathlib

__version__ = "0.1.0"

_SOURCE_TREE = pathlib.Path(__file__).resolve().parent.parent / "anticitoyen-vram_b200"
if not _SOURCE_TREE.is_dir():  # pragma: no cover - a broken checkout
    raise ImportError(f"acvram_b200: source tree not found at {_SOURCE_TREE}")
__path__.append(str(_SOURCE_TREE))

_LAZY = {
    "Engine": "acvram_b200.engine",
    "SamplingParams": "acvram_b200.sampling",
    "GenerationOutput": "acvram_b200.engine",
    "load_config": "acvram_b200.config",
    "REGISTRY": "acvram_b200.config",
    "write_random_model": "acvram_b200.weights",
}


def __getattr__(name: str):
    where = _LAZY.get(name)
    if where is None:
        raise AttributeError(f"module 'acvram_b200' has no attribute {name!r}")
    return getattr(importlib.import_module(where), name)


__all__ = ["__version__", *_LAZY]
