from .pages import PAGE_TOKENS, CacheError, FreeList
from .store import CacheGroup, CacheNeed, SequenceCache

__all__ = ["PAGE_TOKENS", "CacheError", "FreeList", "CacheGroup", "CacheNeed", "SequenceCache"]
