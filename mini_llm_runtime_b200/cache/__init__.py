from .allocator import OutOfPages, PoolAllocator
from .manager import CacheGroup, CacheManager, CacheStats, RequestCache
from .slots import SLOT_WORDS, read_record, slot_record

__all__ = ["CacheGroup", "CacheManager", "CacheStats", "OutOfPages", "PoolAllocator", "RequestCache",
           "SLOT_WORDS", "read_record", "slot_record"]
