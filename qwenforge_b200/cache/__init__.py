from .allocators import CacheFull, CacheMisuse, PageAllocator, SlotAllocator
from .cache import (PAGE_TOKENS, KvGroup, KvNeed, KvSite, SequenceCache, StateGroup, StateNeed, StateSite, round_up)

__all__ = [
    "CacheFull", "CacheMisuse", "PageAllocator", "SlotAllocator", "PAGE_TOKENS", "KvGroup", "KvNeed", "KvSite",
    "SequenceCache", "StateGroup", "StateNeed", "StateSite", "round_up",
]
