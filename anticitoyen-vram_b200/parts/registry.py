"""Registries of part kinds.  A part is registered under a name and built from a
``PartSpec``; registering needs no change to any file of the package."""

from __future__ import annotations

from typing import Callable

from .plan import PartSpec

MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS,
           "block": BLOCKS}


def register(category: str, name: str) -> Callable[[type], type]:
    """Class decorator: ``@register("mixer", "attention")``."""
    table = _TABLES[category]

    def deco(cls: type) -> type:
        table[name] = cls
        cls.kind = name
        return cls

    return deco


def build(category: str, spec: PartSpec, hidden_size: int):
    table = _TABLES[category]
    cls = table.get(spec.kind)
    if cls is None:
        raise KeyError(f"no {category} part named '{spec.kind}'; known: {', '.join(sorted(table)) or 'none'}")
    return cls(hidden_size=hidden_size, **spec.params)
