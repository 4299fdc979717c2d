"""Slots, paged keys and values, and per-sequence state."""
from .allocators import CacheError, FreeList, pages_for
from .sequence_cache import PAGE, CacheView, KVRequest, SequenceCache, StateRequest

__all__ = ["CacheError", "FreeList", "pages_for", "PAGE", "CacheView", "KVRequest", "SequenceCache", "StateRequest"]
