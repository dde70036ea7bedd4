"""A decoder put together from a ModelPlan: embedding, scheduled blocks, final norm, head."""

from __future__ import annotations

import torch

from ..cache.manager import CachePlan
from ..kernels import ops
from ..parts import BLOCKS, CacheView, ModelPlan, Runtime, build
from ..parts.linear import Linear
from ..weights.needs import TensorNeed


class DecoderModel:
    """embed -> blocks in ``plan.schedule`` order -> final norm of the wanted rows -> logits in float32
    (acvram/engine/model.py:143-307).  Knows the plan, not the architecture."""

    def __init__(self, plan: ModelPlan) -> None:
        self.plan = plan
        self.blocks = []
        for spec in plan.layers:
            cls = BLOCKS.get(spec.block)
            if cls is None:
                raise KeyError(f"no block arrangement named '{spec.block}'; known: {', '.join(sorted(BLOCKS))}")
            self.blocks.append(cls(spec, plan.hidden_size))
        self.final_norm = build("norm", plan.final_norm, plan.hidden_size)
        self.rt: Runtime | None = None
        for e in plan.schedule:
            if not 0 <= e.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {e.layer}, the plan has {len(self.blocks)}")

    # ------------------------------------------------------------------ weights
    def tensor_needs(self) -> dict[str, TensorNeed]:
        plan = self.plan
        needs = {plan.embedding_name: TensorNeed((plan.vocab_size, plan.hidden_size), "embedding")}
        for block in self.blocks:
            for name, need in block.tensor_needs().items():
                needs[block.prefix + name] = need
        for name, need in self.final_norm.tensor_needs().items():
            needs[plan.final_norm_prefix + name] = need
        # a tied head reads the embedding; a file that still carries the head's tensor is accepted
        needs[plan.head_name] = TensorNeed((plan.vocab_size, plan.hidden_size), "matrix", optional=plan.tied_head)
        return needs

    def load(self, tensors: dict[str, torch.Tensor], rt: Runtime) -> None:
        plan = self.plan
        self.rt = rt
        self.embedding = tensors[plan.embedding_name].to(device=rt.device, dtype=rt.dtype).contiguous()
        for block in self.blocks:
            p = block.prefix
            block.load({n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}, rt)
        p = plan.final_norm_prefix
        self.final_norm.load({n[len(p):]: t for n, t in tensors.items() if n.startswith(p)}, rt)
        if plan.tied_head:
            self.head = Linear(self.embedding)  # the same storage, no copy
        else:
            self.head = Linear(tensors[plan.head_name].to(device=rt.device, dtype=rt.dtype))

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                key = obj.untyped_storage().data_ptr()
                if key not in seen:
                    seen.add(key)
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, Linear):
                visit(obj.weight)
            elif hasattr(obj, "__dict__") and not isinstance(obj, (type, Runtime, ModelPlan)):
                for v in vars(obj).values():
                    visit(v)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)

        visit(self)
        return total

    # ------------------------------------------------------------------ cache
    def cache_plan(self) -> CachePlan:
        needs = [None] * self.plan.num_cache_slots
        for e in self.plan.schedule:
            if e.cache < 0:
                continue
            need = self.blocks[e.layer].cache_need()
            if e.writes:
                if needs[e.cache] is not None and needs[e.cache] != need:
                    raise ValueError(f"cache slot {e.cache} is written by layers with different needs")
                needs[e.cache] = need
        for e in self.plan.schedule:
            if e.cache >= 0 and not e.writes:
                need = self.blocks[e.layer].cache_need()
                if needs[e.cache] is None or needs[e.cache] != need:
                    raise ValueError(f"layer {e.layer} reads cache slot {e.cache}, which no layer of equal need writes")
        return CachePlan(needs)

    def step_cost(self, q_lens, kv_lens, logit_rows: int, cache_itemsize: int | None = None) -> dict:
        """What one step has to read and compute, summed over the scheduled layers as the parts report it:
        ``weight_bytes`` (each weight once; a layer that runs twice reads its weights twice), ``cache_bytes`` of the
        requests (``q_lens`` new tokens each, ``kv_lens`` held after the step), and ``flops`` of the products, the
        mixing and the head at ``logit_rows`` rows."""
        T = sum(q_lens)
        itemsize = cache_itemsize or self.rt.dtype.itemsize
        weight_bytes = self.head.weight_bytes() + self.final_norm.weight_bytes()
        cache_bytes, flops = 0, self.head.flops(logit_rows)
        for e in self.plan.schedule:
            block = self.blocks[e.layer]
            weight_bytes += block.weight_bytes()
            flops += block.flops(T)
            mixer = getattr(block, "mixer", None)
            if mixer is not None and e.cache >= 0:
                flops += mixer.mixing_flops(q_lens, kv_lens)
                cache_bytes += mixer.cache_bytes_read(q_lens, kv_lens, itemsize)
        return {"weight_bytes": weight_bytes, "cache_bytes": cache_bytes, "flops": flops}

    def uncapturable_parts(self) -> list[str]:
        """Kinds of the parts whose ``capturable`` is false (their forward cannot run inside a CUDA graph)."""
        out = []
        for block in self.blocks:
            for part in (block, *vars(block).values()):
                if getattr(part, "capturable", True) is False and getattr(part, "kind", "?") not in out:
                    out.append(getattr(part, "kind", "?"))
        return out

    def metadata_providers(self) -> dict:
        """{key: a mixer that makes the per-step data its kind needs}: one for each distinct ``metadata_key``."""
        out = {}
        for block in self.blocks:
            mixer = getattr(block, "mixer", None)
            key = getattr(mixer, "metadata_key", None)
            if key is not None and key not in out:
                out[key] = mixer
        return out

    # ------------------------------------------------------------------ the step
    def forward(self, ctx, storage) -> torch.Tensor:
        """Run the step's tokens through every scheduled layer; logits float32 [R, V] at ctx.logit_rows."""
        rt = self.rt
        plan = self.plan
        x = torch.empty((ctx.num_tokens, plan.hidden_size), device=rt.device, dtype=rt.dtype)
        ops.embed(self.embedding, ctx.tokens, x)
        delta = None
        cplan = storage.manager.plan
        for e in plan.schedule:
            view = None
            if e.cache >= 0:
                g = cplan.group_of_slot[e.cache]
                if cplan.groups[g].kind == "paged":
                    k, v = storage.pages(e.cache)
                    view = CacheView(g, e.writes, k_pages=k, v_pages=v)
                else:
                    view = CacheView(g, e.writes, state=storage.state(e.cache))
            x, delta = self.blocks[e.layer].forward(x, delta, ctx, view)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, plan.vocab_size), device=rt.device, dtype=torch.float32)
        h = self.final_norm.forward(x, delta, rows=ctx.logit_rows)
        return self.head(h, out_dtype=torch.float32)
