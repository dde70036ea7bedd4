"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import CacheView, Runtime
from .plan import LayerSpec
from .registry import build, register


@register("block", "prenorm")
class PreNormBlock:
    """x += mixer(norm(x)); x += feed_forward(norm(x)) (acvram/engine/couches.py:404-425).

    The residual travels as (x, delta): the sum x + delta is made inside the next
    norm's kernel, as the reference's deferred-residual path does
    (acvram/engine/couches.py:427-443), so the stream is read and written once per
    sub-block."""

    def __init__(self, spec: LayerSpec, hidden_size: int) -> None:
        self.prefix = spec.prefix
        self.pre_mixer, self.pre_ff = spec.norm_prefixes
        self.input_norm = build("norm", spec.norm, hidden_size)
        self.post_norm = build("norm", spec.norm, hidden_size)
        self.mixer = build("mixer", spec.mixer, hidden_size)
        self.feed_forward = build("feed_forward", spec.feed_forward, hidden_size)

    def tensor_needs(self):
        needs = {}
        for name, need in self.input_norm.tensor_needs().items():
            needs[self.pre_mixer + name] = need
        for name, need in self.post_norm.tensor_needs().items():
            needs[self.pre_ff + name] = need
        needs.update(self.mixer.tensor_needs())
        needs.update(self.feed_forward.tensor_needs())
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        sub = lambda p: {n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}
        self.input_norm.load(sub(self.pre_mixer), rt)
        self.post_norm.load(sub(self.pre_ff), rt)
        self.mixer.load(tensors, rt)
        self.feed_forward.load(tensors, rt)

    def cache_need(self):
        return self.mixer.cache_need()

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in (self.input_norm, self.post_norm, self.mixer, self.feed_forward))

    def flops(self, num_tokens: int) -> float:
        return self.mixer.flops(num_tokens) + self.feed_forward.flops(num_tokens)

    def forward(self, x, delta, ctx, cache: CacheView | None):
        h = self.input_norm.forward(x, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.post_norm.forward(x, a)
        return x, self.feed_forward.forward(h, ctx)
