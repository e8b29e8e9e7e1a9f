"""Cache manager: pages with block tables per request, groups of layers with
different needs, and slots for fixed-size per-request state."""

from .manager import (CacheManager, CacheNeed, NoFreeSlot, PagedKVNeed, PerRequestNeed, PerTokenNeed,
                      StateNeed)
from .pages import OutOfPages, PageAccountingError, PagePool

__all__ = [
    "CacheManager", "CacheNeed", "NoFreeSlot", "PagedKVNeed", "PerRequestNeed", "PerTokenNeed", "StateNeed",
    "OutOfPages", "PageAccountingError", "PagePool",
]
