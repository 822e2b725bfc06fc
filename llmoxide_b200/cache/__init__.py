"""The cache: slots, pages and lengths on the host; keys, values and the
per-sequence state area on the device."""

from .allocator import PAGE, CacheAllocator, pages_for
from .storage import Cache, CacheEntryView, KVNeed, StateNeed

__all__ = ["PAGE", "CacheAllocator", "pages_for", "Cache", "CacheEntryView", "KVNeed", "StateNeed"]
