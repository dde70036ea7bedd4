"""Arrangements of a layer's parts."""

from __future__ import annotations

import torch

from ..kernels import ops
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
        # Small decode steps can run the whole layer as one persistent kernel (csrc/decode_layer.cu).  Off unless asked
        # for: measured on a B200 at the layer sizes of Qwen3-8B it is slower than the seven separate launches (a step's
        # time goes to the chain of dependent phases, which one kernel does not shorten).
        self.fuse_decode = False

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

    def _fused_decode(self, x, delta, ctx, cache: CacheView | None):
        """A step of up to 16 one-token requests in bfloat16 runs the whole layer as one persistent kernel, when the
        parts are of the kinds that kernel knows (each part says so itself: ``decode_layer_spec``) and the sizes fit;
        None otherwise, and the parts run one by one."""
        if x.dtype != torch.bfloat16 or cache is None or not cache.writes or ctx.max_q_len != 1:
            return None
        T = x.shape[0]
        if T > ops.DECODE_LAYER_TOKENS or T != ctx.num_seqs:
            return None
        specs = [getattr(part, "decode_layer_spec", lambda: None)()
                 for part in (self.input_norm, self.post_norm, self.mixer, self.feed_forward)]
        if any(s is None for s in specs):
            return None
        n1, n2, m, f = specs
        if n1["eps"] != n2["eps"] or cache.k_pages is None:
            return None
        if not ops.decode_layer_takes(T, x.shape[1], f["intermediate_size"], m["num_heads"], m["num_kv_heads"], m["head_dim"],
                                      cache.k_pages.shape[2], m["window"]):
            return None
        work = ctx.work.get(m["metadata_key"], {})
        out = torch.empty_like(x)
        ops.decode_layer(x, delta, out, n1["weight"], n2["weight"], n1["eps"], m["w_qkv"], m["w_o"], f["w_gate_up_pairs"],
                         f["w_down"], m["q_norm"], m["k_norm"], m["qk_eps"], m["cos_sin"], m["num_heads"], m["num_kv_heads"],
                         m["head_dim"], m["scale"], ctx.positions, ctx.seq_of_token, ctx.kv_len, ctx.block_tables[cache.group],
                         ctx.table_rows, cache.k_pages, cache.v_pages, int(work.get("max_dec_kv", 0)))
        return x, out

    def forward(self, x, delta, ctx, cache: CacheView | None):
        if self.fuse_decode:
            fused = self._fused_decode(x, delta, ctx, cache)
            if fused is not None:
                return fused
        h = self.input_norm.forward(x, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.post_norm.forward(x, a)
        return x, self.feed_forward.forward(h, ctx)
