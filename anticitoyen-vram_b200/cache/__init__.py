"""Cache manager (host bookkeeping) and cache storage (device tensors)."""

from .manager import (CacheAccountingError, CacheManager, CachePlan, OutOfPages, PagedGroup, PagedNeed, PagePool,
                      StateGroup, StateNeed)

__all__ = ["CacheAccountingError", "CacheManager", "CachePlan", "CacheStorage", "OutOfPages", "PagedGroup",
           "PagedNeed", "PagePool", "StateGroup", "StateNeed"]


def __getattr__(name):
    if name == "CacheStorage":  # needs torch; the bookkeeping does not
        from .storage import CacheStorage
        return CacheStorage
    raise AttributeError(name)
