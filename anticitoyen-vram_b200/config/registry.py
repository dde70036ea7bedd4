"""One registry from the architecture's name in config.json to its model family.

A family is the pair (configuration class, plan builder).  The plan builder turns
a typed configuration into a ``ModelPlan`` (acvram_b200.parts.plan): the list of
layers, each naming its parts, and the order in which they run.  The reference
maps ``architectures[0]`` through an alias table and falls back to "llama" when
the name is unknown (acvram/engine/config.py:634-671, 889); here an unknown name
is an error that lists what is built.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class ModelFamily:
    name: str
    config_cls: type
    build_plan: Callable[[Any], Any]


REGISTRY: dict[str, ModelFamily] = {}


def register_architecture(name: str, config_cls: type, build_plan: Callable[[Any], Any]) -> ModelFamily:
    """Add (or replace) an architecture.  ``config_cls`` needs ``from_dict``."""
    family = ModelFamily(name, config_cls, build_plan)
    REGISTRY[name] = family
    return family


def _ensure_builtin() -> None:
    # The built-in families register themselves when their module is imported.
    from .. import models  # noqa: F401


def family_of(cfg: Mapping[str, Any]) -> ModelFamily:
    _ensure_builtin()
    archs = cfg.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config key 'architectures' must be a non-empty list of names")
    family = REGISTRY.get(archs[0])
    if family is None:
        raise ConfigError(
            f"architecture '{archs[0]}' is not built; known: {', '.join(sorted(REGISTRY)) or 'none'}")
    return family


def load_config(path: str | os.PathLike):
    """Read ``config.json`` (file or folder) into the typed configuration of its architecture."""
    cfg = read_config_json(path)
    return family_of(cfg).config_cls.from_dict(cfg)
