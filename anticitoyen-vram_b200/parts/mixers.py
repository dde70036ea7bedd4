"""Token mixers.  Attention is the one this architecture has."""

from __future__ import annotations

import torch

from ..cache.manager import PagedNeed
from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import CacheView, Mixer, Runtime
from .linear import Linear
from .plan import PartSpec
from .registry import build, register


@register("mixer", "attention")
class Attention(Mixer):
    """Grouped-query attention over the paged cache, with optional per-head RMS norm
    of q and k before the position encoding (acvram/engine/attention.py:142-145,
    290-365).  q-head h reads kv-head h // (heads/kv_heads); scale defaults to
    head_dim^-1/2 (acvram/engine/attention.py:149-151); ``window`` > 0 limits a query
    to the last ``window`` keys.  Tensor names are the Hugging Face ones, kept by the
    reference (acvram/engine/loader.py:1013-1023)."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PartSpec,
                 qk_norm_eps: float | None = None, scale: float | None = None, window: int = 0,
                 prefix: str = "self_attn.") -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.qk_norm_eps = qk_norm_eps
        self.window = int(window)
        self.prefix = prefix
        self.position = build("position", position, hidden_size)
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim

    def cache_need(self):
        return PagedNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_needs(self):
        H = self.hidden_size
        needs = {
            self.prefix + "q_proj.weight": TensorNeed((self.q_size, H)),
            self.prefix + "k_proj.weight": TensorNeed((self.kv_size, H)),
            self.prefix + "v_proj.weight": TensorNeed((self.kv_size, H)),
            self.prefix + "o_proj.weight": TensorNeed((H, self.q_size)),
        }
        if self.qk_norm_eps is not None:
            needs[self.prefix + "q_norm.weight"] = TensorNeed((self.head_dim,), "norm")
            needs[self.prefix + "k_norm.weight"] = TensorNeed((self.head_dim,), "norm")
        for name, need in self.position.tensor_needs().items():
            needs[self.prefix + name] = need
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda n: tensors[n].to(device=rt.device, dtype=rt.dtype)
        self.qkv = Linear.stacked([w(self.prefix + "q_proj.weight"), w(self.prefix + "k_proj.weight"),
                                   w(self.prefix + "v_proj.weight")])
        self.o = Linear(w(self.prefix + "o_proj.weight"))
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            f = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32).contiguous()
            self.q_norm, self.k_norm = f(self.prefix + "q_norm.weight"), f(self.prefix + "k_norm.weight")
        self.position.load({n[len(self.prefix):]: t for n, t in tensors.items() if n.startswith(self.prefix)}, rt)

    def forward(self, h, ctx, cache: CacheView):
        NH, NKV, D = self.num_heads, self.num_kv_heads, self.head_dim
        table = ctx.block_tables[cache.group]
        kp, vp = (cache.k_pages, cache.v_pages) if cache.writes else (None, None)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rotary = self.position.rotary_table()
        if rotary is not None and ops.gemm_tc_qkv_takes(h, self.qkv.weight, D, rotary, kp):
            # a few tokens: norm, rotation and append ride on the projection's kernel as its tile leaves
            qkv = torch.empty((h.shape[0], self.qkv.out_features), device=h.device, dtype=h.dtype)
            ops.gemm_tc_qkv(h, self.qkv.weight, qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                            ctx.seq_of_token, table, kp, vp, static_weights=True)
        elif rotary is not None:
            qkv = self.qkv(h)
            ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                                    ctx.seq_of_token, table if kp is not None else None, kp, vp)
        else:
            # another position encoding: norm, then the part's own change of q and k, then the append
            qkv = self.qkv(h)
            if self.q_norm is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, None, ctx.positions,
                                        ctx.seq_of_token, None, None, None)
            T = qkv.shape[0]
            self.position.apply(qkv[:, :self.q_size].view(T, NH, D),
                                qkv[:, self.q_size:self.q_size + self.kv_size].view(T, NKV, D), ctx)
            if kp is not None:
                ops.qk_norm_rope_append(qkv, NH, NKV, D, None, None, 0.0, None, ctx.positions, ctx.seq_of_token,
                                        table, kp, vp)
        out = torch.empty((qkv.shape[0], self.q_size), device=h.device, dtype=h.dtype)
        ops.attention(qkv, out, cache.k_pages, cache.v_pages, ctx, table, NH, NKV, D, self.scale, self.window)
        return self.o(out)
