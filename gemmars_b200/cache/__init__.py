from .pool import (PAGE_SIZE, CacheError, KVGroup, KVNeed, PageAllocator, SequenceCache, SlotAllocator,  # noqa: F401
                   StateGroup, StateNeed)
