"""Sequence slots, paged key/value storage per layer group, fixed-size per-sequence state."""
from .allocators import CacheError, CacheFull, FreeList
from .sequence_cache import (CacheStore, KVGroup, KVRequest, KVView, PAGE_SIZE, PagedStore, SequenceCache,
                             StateRequest, StateStore, StateView, register_cache_store)

__all__ = ["CacheError", "CacheFull", "CacheStore", "FreeList", "KVGroup", "KVRequest", "KVView", "PAGE_SIZE",
           "PagedStore", "SequenceCache", "StateRequest", "StateStore", "StateView", "register_cache_store"]
