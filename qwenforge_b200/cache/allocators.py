"""Host-side bookkeeping of the cache: which sequence slots and which storage pages are free.

Both allocators refuse what would corrupt the cache silently: taking more than is free,
giving back something that is not held, giving it back twice.
"""
from __future__ import annotations


class CacheFull(RuntimeError):
    """The request does not fit: no free slot, or not enough free pages."""


class CacheMisuse(RuntimeError):
    """A slot or page was released twice, or used while not held."""


class SlotAllocator:
    """Slots 0..n-1, one per live sequence. Freed slots are handed out again, lowest first."""

    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("the cache needs at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))  # pop() yields the lowest
        self._held = [False] * n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._held[slot]

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def give_back(self, slot: int) -> None:
        if not self.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not held (released twice, or never taken)")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


class PageAllocator:
    """Pages 0..n-1 of one group's storage."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a cache group needs at least one page")
        self.n_pages = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self, count: int) -> list[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} cache pages wanted, {len(self._free)} of {self.n_pages} free")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._held[p] = True
        return pages

    def give_back(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not (0 <= p < self.n_pages) or not self._held[p]:
                raise CacheMisuse(f"page {p} is not held (released twice, or never taken)")
            self._held[p] = False
        self._free.extend(sorted(pages, reverse=True))
