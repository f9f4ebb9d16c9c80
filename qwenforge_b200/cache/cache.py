"""The sequence cache: what a model keeps between steps, per sequence.

A *slot* stands for one live sequence. It is taken when the sequence starts, holds the
sequence's own length, and is given back when the sequence ends; the next sequence that
starts takes it again.

What is kept per slot is declared by the model's mixers, one *need* per schedule entry:

  KvNeed     keys and values of every position (window 0) or of the last `window` positions.
             Storage is handed out in pages of PAGE_TOKENS positions, so a sequence holds
             ceil(length / PAGE_TOKENS) pages and nothing more: the cache is sized by the
             number of live tokens, not by slots x longest sequence.
  StateNeed  a tensor of fixed shape per sequence (a recurrent state, a running statistic),
             zeroed when the slot is taken.

Entries with the same need share a *group*; each group has storage of its own (its own
pages, page table and page allocator). A group with a window gives pages back as soon as
every position on them has left the window, so in steady state a sequence holds about
window / PAGE_TOKENS + 1 pages there.

The state that decoding itself keeps per sequence (latest token, position, step count, budget)
lives in the decode graph's own device buffers (`engine/graphs.py`); this cache holds only what
the model's mixers declare.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .allocators import CacheFull, CacheMisuse, PageAllocator, SlotAllocator

PAGE_TOKENS = 64

def round_up(n: int, multiple: int) -> int:
    return (n + multiple - 1) // multiple * multiple


@dataclass(frozen=True)
class KvNeed:
    kv_heads: int
    head_dim: int
    window: int = 0  # 0: every earlier position


@dataclass(frozen=True)
class StateNeed:
    shape: tuple
    dtype: torch.dtype = torch.float32


class KvSite:
    """One schedule entry's view of its group: its own storage, the group's shared page table."""

    def __init__(self, group: "KvGroup", index: int):
        self.group = group
        self.storage = group.storage[index]  # [pages, 2, kv_heads, PAGE_TOKENS, head_dim]
        self.table = group.table
        self.kv_heads = group.need.kv_heads
        self.head_dim = group.need.head_dim
        self.window = group.need.window


class KvGroup:
    def __init__(self, need: KvNeed, entries: Sequence[int], n_pages: int, n_slots: int, pages_per_seq: int,
                 dtype: torch.dtype, device):
        self.need = need
        self.entries = list(entries)
        self.pages = PageAllocator(n_pages)
        self.pages_per_seq = pages_per_seq
        # zeroed once: no kernel reads beyond a sequence's length, stale data is finite anyway
        self.storage = torch.zeros((len(self.entries), n_pages, 2, need.kv_heads, PAGE_TOKENS, need.head_dim),
                                   dtype=dtype, device=device)
        self.table = torch.full((n_slots, pages_per_seq), -1, dtype=torch.int32, device=device)
        self._host_table = torch.full((n_slots, pages_per_seq), -1, dtype=torch.int32)
        self._held: list[dict[int, int]] = [dict() for _ in range(n_slots)]  # slot -> {logical page: page id}
        self._dirty: set[int] = set()

    def pages_missing(self, slot: int, first_pos: int, end_pos: int) -> list[int]:
        """Logical pages covering positions [first_pos, end_pos) that the slot does not hold."""
        if end_pos <= first_pos:
            return []
        held = self._held[slot]
        return [lp for lp in range(first_pos // PAGE_TOKENS, (end_pos - 1) // PAGE_TOKENS + 1) if lp not in held]

    def first_needed(self, length: int) -> int:
        """Lowest position that a query at position >= length can still see."""
        return max(0, length - self.need.window + 1) if self.need.window > 0 else 0

    def grant(self, slot: int, logical_pages: Sequence[int]) -> None:
        ids = self.pages.take(len(logical_pages))
        for lp, page in zip(logical_pages, ids):
            if lp >= self.pages_per_seq:
                self.pages.give_back(ids)
                raise CacheFull(f"position {lp * PAGE_TOKENS} is beyond the cache's longest sequence "
                                f"({self.pages_per_seq * PAGE_TOKENS} positions)")
            self._held[slot][lp] = page
            self._host_table[slot, lp] = page
        if logical_pages:
            self._dirty.add(slot)

    def trim(self, slot: int, length: int) -> None:
        """Give back pages all of whose positions have left the window of every later query."""
        if self.need.window <= 0:
            return
        keep_from = self.first_needed(length) // PAGE_TOKENS
        gone = [lp for lp in self._held[slot] if lp < keep_from]
        if gone:
            self.pages.give_back([self._held[slot].pop(lp) for lp in gone])
            for lp in gone:
                self._host_table[slot, lp] = -1
            self._dirty.add(slot)

    def release(self, slot: int) -> None:
        held = self._held[slot]
        if held:
            self.pages.give_back(list(held.values()))
            held.clear()
            self._host_table[slot].fill_(-1)
            self._dirty.add(slot)

    def pages_held(self, slot: int) -> int:
        return len(self._held[slot])

    def flush(self) -> None:
        """Bring the device page table up to date with the host's (rows that changed since the last call)."""
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        if len(rows) == 1 or rows[-1] - rows[0] + 1 == len(rows):
            lo, hi = rows[0], rows[-1] + 1
            # through a copy of the rows: `trim` and `release` may rewrite the host table as soon as this returns,
            # and a copy from that pageable snapshot has left the host when the call returns
            self.table[lo:hi].copy_(self._host_table[lo:hi].clone())
        else:
            index = torch.tensor(rows, dtype=torch.long)
            self.table.index_copy_(0, index.to(self.table.device), self._host_table[index].to(self.table.device))


class StateGroup:
    def __init__(self, need: StateNeed, entries: Sequence[int], n_slots: int, device):
        self.need = need
        self.entries = list(entries)
        self.storage = torch.zeros((len(self.entries), n_slots, *need.shape), dtype=need.dtype, device=device)

    def reset(self, slot: int) -> None:
        self.storage[:, slot].zero_()


class StateSite:
    """One schedule entry's fixed-size state: `storage[slot]` belongs to the sequence in `slot`."""

    def __init__(self, group: StateGroup, index: int):
        self.group = group
        self.storage = group.storage[index]  # [slots, *shape]


class SequenceCache:
    """Slots and groups of one model on one device.

    needs        one entry per schedule entry: KvNeed, StateNeed or None (that entry keeps nothing,
                 or reads another entry's cache)
    max_tokens   the most tokens that live sequences hold at any time, each sequence's count
                 rounded up to PAGE_TOKENS; sizes every KV group
    max_seqs     number of slots
    max_len      the longest sequence a slot can hold (sizes the page tables)
    """

    _serials = 0

    def __init__(self, needs: Sequence[Optional[object]], max_tokens: int, max_seqs: int, max_len: int,
                 dtype: torch.dtype, device):
        self.device = torch.device(device)
        self.dtype = dtype
        SequenceCache._serials += 1
        self.serial = SequenceCache._serials  # tells caches apart for whoever keeps things per cache (captured graphs)
        n_pages = max(1, round_up(max_tokens, PAGE_TOKENS) // PAGE_TOKENS)
        self.n_pages = n_pages
        self.max_seqs = max(1, min(max_seqs, n_pages))
        self.max_len = min(round_up(max_len, PAGE_TOKENS), n_pages * PAGE_TOKENS)
        pages_per_seq = self.max_len // PAGE_TOKENS
        self.slots = SlotAllocator(self.max_seqs)
        self.lengths = [0] * self.max_seqs

        by_need: dict[object, list[int]] = {}
        for entry, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(entry)
        self.kv_groups: list[KvGroup] = []
        self.state_groups: list[StateGroup] = []
        self._sites: dict[int, object] = {}
        for need, entries in by_need.items():
            if isinstance(need, KvNeed):
                group = KvGroup(need, entries, n_pages, self.max_seqs, pages_per_seq, dtype, self.device)
                self.kv_groups.append(group)
                for i, entry in enumerate(entries):
                    self._sites[entry] = KvSite(group, i)
            elif isinstance(need, StateNeed):
                group = StateGroup(need, entries, self.max_seqs, self.device)
                self.state_groups.append(group)
                for i, entry in enumerate(entries):
                    self._sites[entry] = StateSite(group, i)
            else:
                raise TypeError(f"unknown cache need {need!r}")

    # ------------------------------------------------------------------ sites
    def site(self, entry: int):
        """The storage view of schedule entry `entry` (None if it keeps nothing)."""
        return self._sites.get(entry)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """Start a sequence: take a slot with length 0 and zeroed fixed-size state."""
        slot = self.slots.take()
        self.lengths[slot] = 0
        for group in self.state_groups:
            group.reset(slot)
        return slot

    def _check_held(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheMisuse(f"slot {slot} is not held by a live sequence")

    def reserve(self, requests: Sequence[tuple[int, int]]) -> None:
        """Make sure that each (slot, total_length) has pages for positions up to total_length.

        All or nothing: if the pages for all requests together are not free, CacheFull is
        raised and nothing has changed.
        """
        plans = []
        for group in self.kv_groups:
            wanted = 0
            plan = []
            for slot, total in requests:
                self._check_held(slot)
                if total > self.max_len:
                    raise CacheFull(f"a sequence of {total} tokens exceeds the cache's longest sequence ({self.max_len})")
                first = min(group.first_needed(self.lengths[slot]), self.lengths[slot])
                missing = group.pages_missing(slot, first, total)
                wanted += len(missing)
                plan.append((slot, missing))
            if wanted > group.pages.n_free:
                raise CacheFull(f"{wanted} cache pages wanted ({wanted * PAGE_TOKENS} tokens), "
                                f"{group.pages.n_free} of {group.pages.n_pages} free")
            plans.append((group, plan))
        for group, plan in plans:
            for slot, missing in plan:
                group.grant(slot, missing)

    def advance(self, slot: int, n_tokens: int) -> None:
        """The sequence grew by n_tokens (a step wrote them); windowed groups drop what no later query sees."""
        self._check_held(slot)
        self.lengths[slot] += n_tokens
        for group in self.kv_groups:
            group.trim(slot, self.lengths[slot])

    def close(self, slot: int) -> None:
        """End a sequence: its pages and its slot become free."""
        self._check_held(slot)
        for group in self.kv_groups:
            group.release(slot)
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def flush(self) -> None:
        for group in self.kv_groups:
            group.flush()

    # ------------------------------------------------------------------ accounting
    def tokens_free(self) -> int:
        if not self.kv_groups:
            return self.n_pages * PAGE_TOKENS
        return min(g.pages.n_free for g in self.kv_groups) * PAGE_TOKENS

    def live_slots(self) -> list[int]:
        return [s for s in range(self.max_seqs) if self.slots.is_held(s)]

    def read_bytes(self, lengths: Sequence[int]) -> int:
        """Bytes of keys and values that one single-token step reads for sequences of these lengths."""
        total = 0
        for g in self.kv_groups:
            per_token = len(g.entries) * 2 * g.need.kv_heads * g.need.head_dim * g.storage.element_size()
            total += per_token * sum(min(n, g.need.window) if g.need.window > 0 else n for n in lengths)
        return total

    def storage_bytes(self) -> int:
        total = sum(g.storage.numel() * g.storage.element_size() for g in self.kv_groups)
        total += sum(g.storage.numel() * g.storage.element_size() for g in self.state_groups)
        return total
