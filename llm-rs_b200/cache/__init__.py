"""Paged cache: page pools, the manager that owns the bookkeeping, and device storage."""
from .pool import CacheError, OutOfPages, PagePool
from .manager import RELEASED, CacheManager, GroupSpec, NoFreeSlot, RequestRecord, pages_for

__all__ = ["CacheError", "OutOfPages", "PagePool", "RELEASED", "CacheManager", "GroupSpec", "NoFreeSlot",
           "RequestRecord", "pages_for", "plan_groups", "CacheStorage", "LayerCache"]


def __getattr__(name):
    # The storage needs torch; the bookkeeping above does not.
    if name in ("plan_groups", "CacheStorage", "LayerCache"):
        from . import storage
        return getattr(storage, name)
    raise AttributeError(name)
