from .manager import CacheError, CacheManager, FREED, GroupLayout, OutOfPages, PagePool
from .storage import GroupStorage, StateStorage

__all__ = ["CacheError", "CacheManager", "FREED", "GroupLayout", "OutOfPages", "PagePool",
           "GroupStorage", "StateStorage"]
