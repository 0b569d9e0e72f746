from .manager import UNKNOWN_TOKEN, Allocation, CacheManager, CacheSnapshot, CacheStats, GroupPages, GroupSpec, PageCopy, UnknownRequest
from .needs import PagedKVNeed, StateNeed
from .page_pool import OutOfPages, PagePool, chain_hashes, page_hash
from .pools import CachePools, LayerCache, plan_groups

__all__ = [
    "UNKNOWN_TOKEN",
    "Allocation", "CacheManager", "CachePools", "CacheSnapshot", "CacheStats", "GroupPages", "GroupSpec", "LayerCache", "OutOfPages",
    "PageCopy", "PagePool", "PagedKVNeed", "StateNeed", "UnknownRequest", "chain_hashes", "page_hash", "plan_groups",
]
