from .manager import FREED, CacheError, CacheManager, GroupSpec, PageAllocator, RequestCache, SlotAllocator

__all__ = ["FREED", "CacheError", "CacheManager", "GroupSpec", "PageAllocator", "RequestCache", "SlotAllocator"]
