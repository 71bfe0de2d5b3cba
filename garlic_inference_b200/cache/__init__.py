from .allocator import CacheError, GroupTable, PagePool, SlotAllocator
from .paged import (TOKEN_UNIT, EntryRequirement, EntryView, KVRequirement, KVView, PagedCache, StateRequirement,
                    split_requirement)

__all__ = ["CacheError", "GroupTable", "PagePool", "SlotAllocator", "TOKEN_UNIT", "EntryRequirement", "EntryView",
           "KVRequirement", "KVView", "PagedCache", "StateRequirement", "split_requirement"]
