"""Token mixers.  Attention is the one this architecture has."""

from __future__ import annotations

import torch

from ..cache.manager import PagedNeed
from ..kernels import ops
from ..weights.needs import TensorNeed
from .base import CacheView, Mixer, Runtime, StepMetadata
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
    reference (acvram/engine/loader.py:1013-1023).  ``bias``: True, the four projections have
    biases; False, none; None, those that the weight file holds (acvram/engine/loader.py:269-270)."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PartSpec,
                 qk_norm_eps: float | None = None, scale: float | None = None, window: int = 0,
                 prefix: str = "self_attn.", bias: bool | None = None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.qk_norm_eps = qk_norm_eps
        self.window = int(window)
        self.prefix = prefix
        self.bias = bias
        self.position = build("position", position, hidden_size)
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim

    def cache_need(self):
        return PagedNeed(self.num_kv_heads, self.head_dim, self.window)

    # what the attention kernels want of a step beside the generic batch: their work lists.  One set serves every
    # attention layer of a model (the lists depend on the step's requests only), hence one key.
    metadata_key = "attention"

    def step_metadata(self, q_lens, kv_lens, cu_q) -> StepMetadata:
        return StepMetadata(*ops.attention_work(q_lens, kv_lens, cu_q))

    def decode_metadata(self, padded: int, max_kv: int) -> StepMetadata:
        return StepMetadata(*ops.attention_work_decode(padded, max_kv))

    def tensor_needs(self):
        H = self.hidden_size
        needs = {}
        for name, n_out, n_in in (("q_proj.", self.q_size, H), ("k_proj.", self.kv_size, H), ("v_proj.", self.kv_size, H),
                                  ("o_proj.", H, self.q_size)):
            needs.update(Linear.needs(self.prefix + name, n_out, n_in, self.bias))
        if self.qk_norm_eps is not None:
            needs[self.prefix + "q_norm.weight"] = TensorNeed((self.head_dim,), "norm")
            needs[self.prefix + "k_norm.weight"] = TensorNeed((self.head_dim,), "norm")
        for name, need in self.position.tensor_needs().items():
            needs[self.prefix + name] = need
        return needs

    def load(self, tensors, rt: Runtime) -> None:
        w = lambda n: tensors[n].to(device=rt.device, dtype=rt.dtype)
        b = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32) if n in tensors else None
        self.qkv = Linear.stacked([w(self.prefix + "q_proj.weight"), w(self.prefix + "k_proj.weight"),
                                   w(self.prefix + "v_proj.weight")],
                                  [b(self.prefix + "q_proj.bias"), b(self.prefix + "k_proj.bias"), b(self.prefix + "v_proj.bias")])
        self.o = Linear(w(self.prefix + "o_proj.weight"), b(self.prefix + "o_proj.bias"))
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None:
            f = lambda n: tensors[n].to(device=rt.device, dtype=torch.float32).contiguous()
            self.q_norm, self.k_norm = f(self.prefix + "q_norm.weight"), f(self.prefix + "k_norm.weight")
        self.position.load({n[len(self.prefix):]: t for n, t in tensors.items() if n.startswith(self.prefix)}, rt)

    def decode_layer_spec(self):
        """What the fused decode-layer kernel needs of this mixer (it knows rotary positions over the whole head,
        applied by table, and no biases)."""
        rotary = self.position.rotary_table()
        if self.qkv.bias is not None or self.o.bias is not None or rotary is None or rotary.shape[1] != self.head_dim:
            return None
        return {"num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads, "head_dim": self.head_dim,
                "window": self.window, "scale": self.scale, "w_qkv": self.qkv.weight, "w_o": self.o.weight,
                "q_norm": self.q_norm, "k_norm": self.k_norm, "qk_eps": self.qk_norm_eps or 0.0, "cos_sin": rotary,
                "metadata_key": self.metadata_key}

    # ---- cost of a step
    def weight_bytes(self) -> int:
        norms = sum(t.numel() * 4 for t in (self.q_norm, self.k_norm) if t is not None)
        return self.qkv.weight_bytes() + self.o.weight_bytes() + norms

    def flops(self, num_tokens: int) -> float:
        return self.qkv.flops(num_tokens) + self.o.flops(num_tokens)

    def _seen(self, q: int, kv: int) -> float:
        """Keys that the q queries at the end of a context of kv tokens see, summed over the queries."""
        full = q * (kv - q) + q * (q + 1) / 2
        if self.window <= 0:
            return full
        return sum(min(self.window, kv - q + i + 1) for i in range(q))

    def mixing_flops(self, q_lens, kv_lens) -> float:
        return 4.0 * self.num_heads * self.head_dim * sum(self._seen(q, kv) for q, kv in zip(q_lens, kv_lens))

    def cache_bytes_read(self, q_lens, kv_lens, itemsize: int) -> int:
        keys = sum(min(kv, self.window + q - 1) if self.window > 0 else kv for q, kv in zip(q_lens, kv_lens))
        return 2 * keys * self.kv_size * itemsize

    def forward(self, h, ctx, cache: CacheView):
        NH, NKV, D = self.num_heads, self.num_kv_heads, self.head_dim
        table = ctx.block_tables[cache.group]
        rows = ctx.table_rows
        kp, vp = (cache.k_pages, cache.v_pages) if cache.writes else (None, None)
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rotary = self.position.rotary_table()
        if rotary is not None and self.qkv.bias is None and ops.gemm_tc_qkv_takes(h, self.qkv.weight, D, rotary, kp):
            # a few tokens: norm, rotation and append ride on the projection's kernel as its tile leaves
            qkv = torch.empty((h.shape[0], self.qkv.out_features), device=h.device, dtype=h.dtype)
            ops.gemm_tc_qkv(h, self.qkv.weight, qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                            ctx.seq_of_token, table, kp, vp, static_weights=True, table_rows=rows)
        elif rotary is not None:
            qkv = self.qkv(h)
            ops.qk_norm_rope_append(qkv, NH, NKV, D, self.q_norm, self.k_norm, eps, rotary, ctx.positions,
                                    ctx.seq_of_token, table if kp is not None else None, kp, vp, table_rows=rows)
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
                                        table, kp, vp, table_rows=rows)
        out = torch.empty((qkv.shape[0], self.q_size), device=h.device, dtype=h.dtype)
        ops.attention(qkv, out, cache.k_pages, cache.v_pages, ctx, table, NH, NKV, D, self.scale, self.window,
                      work=ctx.work[self.metadata_key])
        return self.o(out)
