from .allocator import OutOfPages, PoolAllocator
from .manager import CacheGroup, CacheManager, CacheStats, RequestCache

__all__ = ["CacheGroup", "CacheManager", "CacheStats", "OutOfPages", "PoolAllocator", "RequestCache"]
