"""The cache's bookkeeping on the host: no slot or page lost, held twice or freed twice (no GPU)."""

import random

import pytest
import torch

from ondeviceinfer_b200.cache import (PAGE_SIZE, CacheCapacityError, IndexAllocator, KVNeed, SequenceCache,
                                      StateNeed, pages_for)


def make_cache(max_tokens=1024, max_seqs=6, needs=None, cache_from=None, **kw):
    needs = needs if needs is not None else [(KVNeed(2, 16),)] * 3
    cache_from = cache_from if cache_from is not None else [None] * len(needs)
    return SequenceCache(needs, cache_from, dtype=torch.float32, device="cpu", max_tokens=max_tokens,
                         max_seqs=max_seqs, **kw)


def test_index_allocator_refuses_misuse():
    a = IndexAllocator(3, "slot")
    got = [a.take(), a.take(), a.take()]
    assert sorted(got) == [0, 1, 2]
    with pytest.raises(CacheCapacityError):
        a.take()
    a.give_back(1)
    with pytest.raises(ValueError):
        a.give_back(1)
    with pytest.raises(ValueError):
        a.give_back(7)
    assert a.take() == 1
    a.check()


def test_slots_are_reused_and_lengths_start_at_zero():
    cache = make_cache()
    s = [cache.alloc() for _ in range(6)]
    assert sorted(s) == list(range(6))
    with pytest.raises(CacheCapacityError):
        cache.alloc()
    cache.reserve([s[2]], [100])
    cache.advance([s[2]], [100])
    assert cache.length(s[2]) == 100
    cache.free(s[2])
    with pytest.raises(ValueError):
        cache.free(s[2])
    with pytest.raises(ValueError):
        cache.length(s[2])
    again = cache.alloc()
    assert again == s[2] and cache.length(again) == 0
    cache.check()


def test_pages_follow_lengths_and_capacity_counts_rounded_tokens():
    cache = make_cache(max_tokens=4 * PAGE_SIZE, max_seqs=4)
    a, b = cache.alloc(), cache.alloc()
    cache.reserve([a, b], [1, PAGE_SIZE + 1])       # 1 + 2 pages
    cache.advance([a, b], [1, PAGE_SIZE + 1])
    group = cache.kv_groups[0]
    assert [len(group.slot_pages[s]) for s in (a, b)] == [1, 2]
    assert cache.tokens_held == 3 * PAGE_SIZE
    cache.reserve([a], [PAGE_SIZE - 1])             # still inside a's first page
    cache.advance([a], [PAGE_SIZE - 1])
    assert len(group.slot_pages[a]) == 1
    cache.reserve([a], [1])                         # the fourth page
    cache.advance([a], [1])
    with pytest.raises(CacheCapacityError) as error:
        cache.reserve([b], [PAGE_SIZE])
    assert "capacity" in str(error.value)
    assert [len(group.slot_pages[s]) for s in (a, b)] == [2, 2]   # nothing was taken by the failed call
    cache.free(a)
    cache.reserve([b], [PAGE_SIZE])
    cache.check()


def test_reserve_is_all_or_nothing_across_sequences():
    cache = make_cache(max_tokens=3 * PAGE_SIZE, max_seqs=3)
    a, b = cache.alloc(), cache.alloc()
    with pytest.raises(CacheCapacityError):
        cache.reserve([a, b], [2 * PAGE_SIZE, 2 * PAGE_SIZE])
    assert cache.kv_groups[0].pages.held_count == 0
    with pytest.raises(ValueError):
        cache.reserve([a, a], [1, 1])
    cache.check()


def test_groups_by_need_have_storage_of_their_own():
    full, window, state = KVNeed(2, 16), KVNeed(2, 16, window=40), StateNeed((4, 8))
    needs = [(full,), (window,), (full,), (window, ), (state,), ()]
    cache = make_cache(needs=needs, cache_from=[None, None, None, None, None, 2], max_tokens=1024, max_seqs=4,
                       max_step_tokens=32)
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1
    g_full = next(g for g in cache.kv_groups if g.need.window is None)
    g_win = next(g for g in cache.kv_groups if g.need.window == 40)
    assert g_full.owners == [0, 2] and g_win.owners == [1, 3]
    assert g_full.pool.shape == (2, 2, 16 + 1, 2, PAGE_SIZE, 16)   # one more page for padding rows
    assert g_full.pool.data_ptr() != g_win.pool.data_ptr()
    assert g_full.ring_pages == 0 and g_win.ring_pages == pages_for(40 + 32 - 1) + 1
    assert cache.max_step_tokens == 32
    # entry 5 reads entry 2's cache and writes nothing
    assert cache.view(5).keys.data_ptr() == cache.view(2).keys.data_ptr() and not cache.view(5).writes_kv
    assert cache.view(2).writes_kv and cache.view(0).keys.data_ptr() != cache.view(2).keys.data_ptr()
    assert cache.view(4).state.shape == (4 + 1, 4, 8) and cache.view(4).keys is None
    s = cache.alloc()
    cache.reserve([s], [500])
    cache.advance([s], [500])
    assert len(g_full.slot_pages[s]) == pages_for(500) and len(g_win.slot_pages[s]) == g_win.ring_pages
    cache.free(s)
    cache.check()


def test_state_rows_are_zeroed_when_a_slot_is_taken():
    cache = make_cache(needs=[(StateNeed((3,)),)], max_seqs=2)
    s = cache.alloc()
    cache.view(0).state[s] += 5.0
    cache.free(s)
    t = cache.alloc()
    assert t == s and float(cache.view(0).state[t].abs().sum()) == 0.0


def test_random_traffic_never_loses_or_doubles_anything():
    rng = random.Random(0)
    cache = make_cache(max_tokens=40 * PAGE_SIZE, max_seqs=8)
    live = {}
    for _ in range(2000):
        action = rng.random()
        if action < 0.3 and len(live) < 8:
            live[cache.alloc()] = 0
        elif action < 0.5 and live:
            slot = rng.choice(list(live))
            cache.free(slot)
            del live[slot]
        elif live:
            slot = rng.choice(list(live))
            t = rng.randint(1, 150)
            try:
                cache.reserve([slot], [t])
                cache.advance([slot], [t])
                live[slot] += t
            except CacheCapacityError:
                pass
        cache.check()
        assert {s: cache.length(s) for s in live} == live
        assert cache.kv_groups[0].pages.held_count == sum(pages_for(n) for n in live.values())
    cache.reset()
    cache.check()
    assert cache.kv_groups[0].pages.held_count == 0 and cache.slots.held_count == 0


def test_padding_slot_lies_outside_the_capacity():
    cache = make_cache(max_tokens=2 * PAGE_SIZE, max_seqs=2)
    group = cache.kv_groups[0]
    assert cache.pad_slot == 2 and group.slot_pages[cache.pad_slot] == [group.pad_page] and group.pad_page == 2
    a, b = cache.alloc(), cache.alloc()
    assert cache.pad_slot not in (a, b)
    cache.reserve([a, b], [PAGE_SIZE, PAGE_SIZE])
    assert group.pad_page not in group.slot_pages[a] + group.slot_pages[b]
    assert cache.lengths[cache.pad_slot] == 0
    cache.check()


def test_bad_sizes():
    with pytest.raises(ValueError):
        make_cache(max_tokens=0)
    with pytest.raises(ValueError):
        make_cache(max_seqs=0)
    assert make_cache(max_tokens=65).n_pages == 2
