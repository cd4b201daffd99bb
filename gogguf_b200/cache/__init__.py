"""Sequence slots, paged key/value storage per layer group, fixed-size per-sequence state."""
from .allocators import CacheError, CacheFull, FreeList
from .sequence_cache import KVGroup, KVRequest, KVView, PAGE_SIZE, SequenceCache, StateRequest, StateView

__all__ = ["CacheError", "CacheFull", "FreeList", "KVGroup", "KVRequest", "KVView", "PAGE_SIZE", "SequenceCache",
           "StateRequest", "StateView"]
