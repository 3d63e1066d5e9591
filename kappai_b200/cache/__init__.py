from .spec import PagedKVSpec, StateSpec
from .manager import (CacheManager, PagePool, SlotPool, CacheError, OutOfPages, OutOfSlots, RELEASED)

__all__ = ["PagedKVSpec", "StateSpec", "CacheManager", "PagePool", "SlotPool", "CacheError", "OutOfPages",
           "OutOfSlots", "RELEASED"]
