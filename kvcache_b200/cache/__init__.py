from .manager import CacheGroup, CacheManager, StepCacheView
from .pages import GroupPages, OutOfPages, PageAllocator, pages_for
from .slots import OutOfSlots, SlotAllocator

__all__ = ["CacheGroup", "CacheManager", "StepCacheView", "GroupPages", "OutOfPages", "PageAllocator",
           "pages_for", "OutOfSlots", "SlotAllocator"]
