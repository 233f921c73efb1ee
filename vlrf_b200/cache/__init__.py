from .allocator import CacheError, FreeList
from .sequence_cache import BLOCK_TOKENS, CacheView, KVNeed, SequenceCache, StateNeed

__all__ = ["CacheError", "FreeList", "BLOCK_TOKENS", "CacheView", "KVNeed", "SequenceCache", "StateNeed"]
