from .allocator import CacheFull, IdAllocator
from .kv_cache import CacheGroup, KVCache, SequenceRecord

__all__ = ["CacheFull", "IdAllocator", "CacheGroup", "KVCache", "SequenceRecord"]
