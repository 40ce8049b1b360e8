"""The cache: pages, slots, groups of entries with storage of their own, per-sequence state."""
from .pages import PAGE_TOKENS, CacheError, CacheFull, PagePool, SlotTable, pages_for
from .sequence_cache import KVCacheNeed, KVView, SequenceCache, StateNeed, StateView

__all__ = ["PAGE_TOKENS", "CacheError", "CacheFull", "PagePool", "SlotTable", "pages_for", "KVCacheNeed", "KVView",
           "SequenceCache", "StateNeed", "StateView"]
