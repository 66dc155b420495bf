"""The cache: slots, pages and per-sequence state."""

from .slots import CacheError, FreeList, PageLedger, pages_for
from .store import CacheEntry, KVNeed, SequenceCache, StateNeed

__all__ = ["CacheEntry", "CacheError", "FreeList", "KVNeed", "PageLedger", "SequenceCache", "StateNeed", "pages_for"]
