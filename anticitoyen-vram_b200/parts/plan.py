"""The model as data: which parts make each layer, and in which order layers run.

A ``ModelPlan`` is what an architecture's plan builder makes of its typed
configuration.  Nothing below it knows an architecture's name: a layer is a block
arrangement over a mixer, a feed-forward and norms, each named by ``kind`` and
built from the parameters given here.  Layers may differ from one another, and
``schedule`` may run a layer twice or let a layer read the cache that another
layer writes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """A part by the name it is registered under, with its constructor's parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **more) -> "PartSpec":
        return PartSpec(self.kind, {**self.params, **more})


@dataclass(frozen=True)
class LayerSpec:
    prefix: str          # tensor-name prefix of the layer, e.g. "model.layers.3."
    block: str           # arrangement of the parts, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec       # the norm placed before the mixer and before the feed-forward
    norm_prefixes: tuple[str, str] = ("input_layernorm.", "post_attention_layernorm.")


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache`` is the cache slot its mixer uses (-1: none);
    with ``writes`` false the mixer only reads what another entry wrote there."""

    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    embedding_name: str = "model.embed_tokens.weight"
    final_norm_prefix: str = "model.norm."
    head_name: str = "lm_head.weight"
    tied_head: bool = False
    eos_token_ids: tuple[int, ...] = ()

    @property
    def num_cache_slots(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def default_schedule(num_layers: int) -> tuple[ScheduleEntry, ...]:
    """Each layer once, in order, each with a cache slot of its own."""
    return tuple(ScheduleEntry(i, i, True) for i in range(num_layers))
