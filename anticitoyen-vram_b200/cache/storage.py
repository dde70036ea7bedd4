"""Device memory of the cache groups: page pools and state slots."""

from __future__ import annotations

import torch

from .manager import CacheManager, PagedGroup


class CacheStorage:
    """One tensor for each group.

    Paged group: ``[slots, 2, num_pages, kv_heads, page_size, head_dim]`` (keys at
    index 0 of the second axis, values at 1); a page of one kv-head is contiguous,
    so a tile of keys is a run of ``page_size * head_dim`` elements.  The
    reference keeps ``[num_blocks, 16, kv_heads, head_dim]`` per layer
    (acvram/memory/kvcache.py:463-469).  State group:
    ``[slots, max_requests + 1, *shape]`` (the last slot belongs to nobody: padding rows of a
    fixed-shape batch work on it).  Everything starts at zero, so that a key
    that is masked out never brings a NaN into a product.

    Beside its pages a paged group has its block table on the device, int32
    ``[max_requests + 1, width]``: row r belongs to the request that the manager gave row r, the last row to
    nobody; all entries start at -1 ("no page").  ``max_len`` (tokens) decides the width."""

    def __init__(self, manager: CacheManager, device, dtype: torch.dtype, max_len: int | None = None) -> None:
        self.manager = manager
        self.device = torch.device(device)
        self.dtype = dtype
        self.tensors: list[torch.Tensor] = []
        self.tables: dict[int, torch.Tensor] = {}       # group index -> the group's block table on the device
        for gi, g in enumerate(manager.groups):
            if isinstance(g, PagedGroup):
                shape = (g.num_slots, 2, max(g.pool.num_pages, 1), g.need.num_kv_heads, g.page_size, g.need.head_dim)
                self.tensors.append(torch.zeros(shape, device=self.device, dtype=dtype))
                # a request that keeps all its keys can never hold more pages than the pool has
                tokens = max_len if max_len else g.pool.num_pages * g.page_size
                if g.need.window <= 0:
                    tokens = min(tokens, g.pool.num_pages * g.page_size)
                width = max(1, g.pages_for(tokens))
                self.tables[gi] = torch.full((manager.max_requests + 1, width), -1, device=self.device, dtype=torch.int32)
            else:
                sdtype = getattr(torch, g.need.dtype)
                self.tensors.append(torch.zeros((g.num_slots, g.max_requests + 1, *g.need.shape), device=self.device,
                                                dtype=sdtype))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors)

    @property
    def max_tokens(self) -> int:
        """The longest request that every block table has columns for."""
        return min((t.shape[1] * self.manager.page_size for t in self.tables.values()), default=1 << 30)

    def pages(self, cache_slot: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(keys, values) of a cache slot, each ``[num_pages, kv_heads, page_size, head_dim]``."""
        plan = self.manager.plan
        t = self.tensors[plan.group_of_slot[cache_slot]][plan.index_in_group[cache_slot]]
        return t[0], t[1]

    def state(self, cache_slot: int) -> torch.Tensor:
        """State of a cache slot for all request slots: ``[max_requests + 1, *shape]``."""
        plan = self.manager.plan
        return self.tensors[plan.group_of_slot[cache_slot]][plan.index_in_group[cache_slot]]

    def zero_state(self, group: int, slot: int) -> None:
        self.tensors[group][:, slot].zero_()
