"""The cache manager: paged keys and values per layer group, prefix cache, state slots."""

from paged_kv_serving_b200.cache.manager import GroupSpec, KVCacheManager, PrefixReuse, plan_groups
from paged_kv_serving_b200.cache.pages import (
    NULL_PAGE, AllocatorInvariantError, OutOfPages, PageAllocator, PageStore, RecordingPageStore,
)
from paged_kv_serving_b200.cache.prefix_cache import PrefixCache, PrefixCacheStats, chain_start, extend_chain, hash_chain
from paged_kv_serving_b200.cache.state_slots import StateSlotPool

__all__ = [
    "NULL_PAGE", "AllocatorInvariantError", "GroupSpec", "KVCacheManager", "OutOfPages", "PageAllocator",
    "PageStore", "PrefixCache", "PrefixCacheStats", "PrefixReuse", "RecordingPageStore", "StateSlotPool",
    "chain_start", "extend_chain", "hash_chain", "plan_groups",
]
