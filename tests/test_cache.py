"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; windows give pages back;
a reservation that does not fit changes nothing."""
import random

import pytest
import torch

from qwenforge_b200.cache import (PAGE_TOKENS, CacheFull, CacheMisuse, KvNeed, PageAllocator, SequenceCache,
                                  SlotAllocator, StateNeed)


def test_slot_allocator_never_loses_or_doubles():
    slots = SlotAllocator(5)
    held = set()
    rng = random.Random(0)
    for _ in range(2000):
        if held and (rng.random() < 0.5 or slots.n_free == 0):
            s = rng.choice(sorted(held))
            slots.give_back(s)
            held.remove(s)
        else:
            s = slots.take()
            assert s not in held and 0 <= s < 5
            held.add(s)
        assert slots.n_free + len(held) == 5
    for s in list(held):
        slots.give_back(s)
    assert slots.n_free == 5 and [slots.take() for _ in range(5)] == [0, 1, 2, 3, 4]  # reused, lowest first
    with pytest.raises(CacheFull):
        slots.take()
    slots.give_back(3)
    with pytest.raises(CacheMisuse, match="not held"):
        slots.give_back(3)
    with pytest.raises(CacheMisuse):
        slots.give_back(17)


def test_page_allocator():
    pages = PageAllocator(10)
    a, b = pages.take(4), pages.take(6)
    assert sorted(a + b) == list(range(10)) and pages.n_free == 0
    with pytest.raises(CacheFull):
        pages.take(1)
    pages.give_back(a)
    with pytest.raises(CacheMisuse):
        pages.give_back(a[:1])
    with pytest.raises(CacheFull):
        pages.take(5)
    assert pages.n_free == 4  # a failed request took nothing


def make_cache(window=0, max_tokens=64 * 8, max_seqs=4, max_len=64 * 6):
    needs = [KvNeed(2, 8, 0), KvNeed(2, 8, window), None, StateNeed((3, 2), torch.float32)]
    return SequenceCache(needs, max_tokens, max_seqs, max_len, torch.float32, "cpu")


def test_groups_have_storage_of_their_own():
    cache = make_cache(window=10)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1
    full, windowed = cache.kv_groups
    assert full.storage.data_ptr() != windowed.storage.data_ptr()
    assert full.storage.shape == (1, 8, 2, 2, PAGE_TOKENS, 8)
    assert cache.site(2) is None and cache.site(3).storage.shape == (4, 3, 2)
    same = make_cache(window=0)
    assert len(same.kv_groups) == 1 and same.kv_groups[0].storage.shape[0] == 2  # same need: one group, two sites
    assert same.site(0).storage.data_ptr() != same.site(1).storage.data_ptr()


def test_pages_follow_lengths_and_come_back():
    cache = make_cache()
    group = cache.kv_groups[0]
    a, b = cache.open(), cache.open()
    cache.reserve([(a, 65), (b, 1)])
    assert group.pages_held(a) == 2 and group.pages_held(b) == 1 and group.pages.n_free == 5
    cache.advance(a, 65)
    cache.advance(b, 1)
    cache.reserve([(a, 128), (b, 64)])          # still inside the pages they hold
    assert group.pages.n_free == 5
    cache.reserve([(a, 129)])
    assert group.pages_held(a) == 3
    held = {int(p) for p in group._host_table[a] if p >= 0} | {int(p) for p in group._host_table[b] if p >= 0}
    assert len(held) == 4                        # no page is held twice
    cache.flush()
    assert torch.equal(group.table, group._host_table)
    cache.close(a)
    assert group.pages.n_free == 7 and cache.lengths[a] == 0
    with pytest.raises(CacheMisuse):
        cache.close(a)
    with pytest.raises(CacheMisuse):
        cache.reserve([(a, 5)])
    c = cache.open()
    assert c == a                                # the freed slot is used again
    cache.flush()
    assert int(group.table[c].max()) == -1       # and starts with no pages


def test_reservation_is_all_or_nothing():
    cache = make_cache(max_tokens=64 * 4)
    a, b = cache.open(), cache.open()
    with pytest.raises(CacheFull, match="cache pages wanted"):
        cache.reserve([(a, 130), (b, 100)])      # 3 + 2 pages of 4
    assert all(g.pages.n_free == 4 for g in cache.kv_groups)
    cache.reserve([(a, 130), (b, 64)])
    with pytest.raises(CacheFull, match="longest sequence"):
        cache.reserve([(a, 64 * 6 + 1)])


def test_window_gives_pages_back():
    cache = make_cache(window=70, max_tokens=64 * 8)
    full, windowed = cache.kv_groups
    s = cache.open()
    cache.reserve([(s, 300)])                    # a long prompt in one step holds every page during the step
    assert windowed.pages_held(s) == 5
    cache.advance(s, 300)                        # afterwards only what the next query can see: positions 231..
    assert windowed.pages_held(s) == 2 and full.pages_held(s) == 5
    for length in range(300, 384):
        cache.reserve([(s, length + 1)])
        cache.advance(s, 1)
        assert windowed.pages_held(s) <= 3
        first_visible = length + 1 - 70 + 1
        assert int(windowed._host_table[s, first_visible // 64]) >= 0
    cache.close(s)
    assert windowed.pages.n_free == 8 and full.pages.n_free == 8


def test_fixed_state_is_reset_when_a_slot_is_reused():
    cache = make_cache()
    s = cache.open()
    cache.site(3).storage[s] += 5.0
    cache.close(s)
    t = cache.open()
    assert t == s and float(cache.site(3).storage[t].abs().max()) == 0.0


def test_random_lifetimes_leave_nothing_behind():
    cache = make_cache(window=33, max_tokens=64 * 12, max_seqs=5)
    rng = random.Random(1)
    live = {}
    for _ in range(600):
        action = rng.random()
        if live and action < 0.25:
            s = rng.choice(sorted(live))
            cache.close(s)
            del live[s]
        elif action < 0.5 and cache.slots.n_free:
            try:
                s = cache.open()
                n = rng.randint(1, 150)
                cache.reserve([(s, n)])
                cache.advance(s, n)
                live[s] = n
            except CacheFull:
                cache.close(s)
        elif live:
            s = rng.choice(sorted(live))
            try:
                cache.reserve([(s, live[s] + 1)])
                cache.advance(s, 1)
                live[s] += 1
            except CacheFull:
                pass
        for g in cache.kv_groups:
            held = [int(p) for slot in range(5) for p in g._host_table[slot] if p >= 0]
            assert len(held) == len(set(held)) and len(held) + g.pages.n_free == g.pages.n_pages
        assert cache.lengths[:5] == [live.get(s, 0) for s in range(5)]
    for s in list(live):
        cache.close(s)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups) and cache.slots.n_free == 5
