"""What every architecture's configuration shares: the error type and JSON reading."""

from __future__ import annotations

import json
import os
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this engine cannot run; the message names the key."""


def read_config_json(path: str | os.PathLike) -> dict[str, Any]:
    """Return the dictionary of ``config.json``; ``path`` is the file or its folder."""
    path = os.fspath(path)
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            cfg = json.load(fh)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return merge_generation_stops(cfg, os.path.join(os.path.dirname(os.path.abspath(path)), "generation_config.json"))


def _id_list(value: Any) -> list[int]:
    if isinstance(value, bool):
        return []
    if isinstance(value, int):
        return [value]
    if isinstance(value, (list, tuple)):
        return [v for v in value if isinstance(v, int) and not isinstance(v, bool)]
    return []


def merge_generation_stops(cfg: dict[str, Any], generation_config_path: str) -> dict[str, Any]:
    """The end-of-sequence ids of ``generation_config.json`` beside the model's config.json join those of
    config.json itself: some checkpoints name their end-of-turn token only there, and the reference lets that file
    have its say on the stop tokens (acvram/engine/config.py:816-835).  A file that is absent or unreadable
    changes nothing."""
    if not os.path.isfile(generation_config_path):
        return cfg
    try:
        with open(generation_config_path, "r", encoding="utf-8") as fh:
            gen = json.load(fh)
    except (OSError, json.JSONDecodeError):
        return cfg
    merged = _id_list(cfg.get("eos_token_id")) + (_id_list(gen.get("eos_token_id")) if isinstance(gen, dict) else [])
    if merged:
        cfg = {**cfg, "eos_token_id": sorted(set(merged))}
    return cfg


def take_int(cfg: Mapping[str, Any], key: str, default: int | None = None, *, minimum: int = 1) -> int:
    value = cfg.get(key, default)
    if value is None:
        raise ConfigError(f"config key '{key}' is missing and has no default")
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config key '{key}' must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config key '{key}' must be >= {minimum}, got {value}")
    return value


def take_float(cfg: Mapping[str, Any], key: str, default: float | None = None, *, positive: bool = True) -> float:
    value = cfg.get(key, default)
    if value is None:
        raise ConfigError(f"config key '{key}' is missing and has no default")
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config key '{key}' must be a number, got {value!r}")
    value = float(value)
    if positive and not value > 0.0:
        raise ConfigError(f"config key '{key}' must be > 0, got {value}")
    return value


def take_id_list(cfg: Mapping[str, Any], key: str) -> tuple[int, ...]:
    """``eos_token_id`` may be an integer, a list of integers or absent."""
    value = cfg.get(key)
    if value is None:
        return ()
    if isinstance(value, int) and not isinstance(value, bool):
        return (value,)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
        return tuple(value)
    raise ConfigError(f"config key '{key}' must be an integer or a list of integers, got {value!r}")
