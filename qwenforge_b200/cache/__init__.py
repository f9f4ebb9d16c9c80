from .allocators import CacheFull, CacheMisuse, PageAllocator, SlotAllocator
from .cache import (PAGE_TOKENS, STATE_BUDGET, STATE_FINISHED, STATE_LENGTH, STATE_SEQ_HI, STATE_SEQ_LO, STATE_STEP,
                    STATE_TOKEN, STATE_WORDS, KvGroup, KvNeed, KvSite, SequenceCache, StateGroup, StateNeed, StateSite,
                    round_up)

__all__ = [
    "CacheFull", "CacheMisuse", "PageAllocator", "SlotAllocator", "PAGE_TOKENS", "STATE_BUDGET", "STATE_FINISHED",
    "STATE_LENGTH", "STATE_SEQ_HI", "STATE_SEQ_LO", "STATE_STEP", "STATE_TOKEN", "STATE_WORDS", "KvGroup", "KvNeed",
    "KvSite", "SequenceCache", "StateGroup", "StateNeed", "StateSite", "round_up",
]
