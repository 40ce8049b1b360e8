"""The cache: pages, slots, groups of entries with storage of their own, per-sequence state."""
from .pages import PAGE_TOKENS, CacheError, CacheFull, PagePool, SlotTable, pages_for
from .sequence_cache import (CacheGroup, CacheSizes, KVCacheNeed, KVGroup, KVView, PagedGroup, SequenceCache, StateGroup,
                             StateNeed, StateView, register_cache_group, unregister_cache_group)

__all__ = ["PAGE_TOKENS", "CacheError", "CacheFull", "PagePool", "SlotTable", "pages_for", "CacheGroup", "CacheSizes",
           "KVCacheNeed", "KVGroup", "KVView", "PagedGroup", "SequenceCache", "StateGroup", "StateNeed", "StateView",
           "register_cache_group", "unregister_cache_group"]
