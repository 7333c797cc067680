from .allocator import CacheFull, IdAllocator
from .kinds import CacheKind, cache_kind, register_cache_kind
from .kv_cache import CacheGroup, KVCache, SequenceRecord

__all__ = ["CacheFull", "IdAllocator", "CacheGroup", "CacheKind", "KVCache", "SequenceRecord", "cache_kind",
           "register_cache_kind"]
