"""Pages, block tables, layer groups and state slots (host), and their device tensors."""

from .manager import (NULL_PAGE, CacheManager, GroupState, PagedCacheSpec, PagePool, StateCacheSpec, StateSlots)
from .storage import CacheStorage, bytes_per_page, paged_cache_bytes_per_page

__all__ = ["NULL_PAGE", "CacheManager", "CacheStorage", "GroupState", "PagePool", "PagedCacheSpec",
           "StateCacheSpec", "StateSlots", "bytes_per_page", "paged_cache_bytes_per_page"]
