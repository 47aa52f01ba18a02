from .manager import CacheManager, OutOfPages, OutOfSlots, PagePool, SlotPool

__all__ = ["CacheManager", "OutOfPages", "OutOfSlots", "PagePool", "SlotPool"]
