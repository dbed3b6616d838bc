from .manager import CacheError, CacheManager, GroupSpec, PagePool, SlotPool

__all__ = ["CacheError", "CacheManager", "GroupSpec", "PagePool", "SlotPool"]
