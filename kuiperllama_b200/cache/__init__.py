"""Slots, paged keys and values, and per-sequence state."""
from .allocators import CacheError, FreeList, pages_for
from .sequence_cache import (PAGE, CacheView, KVRequest, PagedGroup, SequenceCache, StateRequest, cache_kind,
                             register_cache_kind)

__all__ = ["CacheError", "FreeList", "pages_for", "PAGE", "CacheView", "KVRequest", "SequenceCache", "StateRequest", "PagedGroup",
           "cache_kind", "register_cache_kind"]
