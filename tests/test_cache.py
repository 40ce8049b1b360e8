"""The cache's bookkeeping: no page or slot is lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from gpullama3.java_b200.cache import (PAGE_TOKENS, CacheError, CacheFull, KVCacheNeed, PagePool, SequenceCache,
                                       SlotTable, StateNeed, pages_for)


def test_page_pool_hands_out_each_page_once():
    pool = PagePool(5)
    a = pool.alloc(3)
    b = pool.alloc(2)
    assert sorted(a + b) == [0, 1, 2, 3, 4] and pool.n_free == 0
    with pytest.raises(CacheFull):
        pool.alloc(1)
    pool.free(a)
    with pytest.raises(CacheError, match="twice"):
        pool.free([a[0]])
    with pytest.raises(CacheError, match="belong"):
        pool.free([17])
    assert sorted(pool.alloc(3)) == sorted(a)


def test_slot_table():
    t = SlotTable(2)
    s0, s1 = t.acquire(), t.acquire()
    assert {s0, s1} == {0, 1}
    with pytest.raises(CacheFull):
        t.acquire()
    t.release(s0)
    with pytest.raises(CacheError):
        t.release(s0)
    with pytest.raises(CacheError):
        t.release(9)
    assert t.acquire() == s0 and t.live_slots() == [0, 1]


def _cache(max_tokens=64 * 6, **kw):
    needs = {0: KVCacheNeed(2, 16), 1: KVCacheNeed(2, 16), 2: KVCacheNeed(1, 32)}
    return SequenceCache(needs, max_tokens=max_tokens, dtype=torch.float32, device="cpu", **kw)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.paged_groups) == 2
    g0, g1 = c.paged_groups
    assert g0.entries == [0, 1] and g1.entries == [2]
    assert tuple(g0.k.shape) == (2, 6, 2, PAGE_TOKENS, 16) and tuple(g1.v.shape) == (1, 6, 1, 32, PAGE_TOKENS)
    v0, v1, v2 = c.view(0), c.view(1), c.view(2)
    assert v0.group == v1.group == 0 and v2.group == 1
    assert v0.k.data_ptr() != v1.k.data_ptr() and tuple(v2.k.shape) == (6, 1, PAGE_TOKENS, 32)
    assert c.bytes_per_token() == 2 * (2 * 2 * 16 + 1 * 1 * 32) * 4


def test_reserve_commit_release_and_reuse():
    c = _cache()
    a, b = c.acquire(), c.acquire()
    c.reserve([(a, 65), (b, 64)])
    c.commit(a, 65)
    c.commit(b, 64)
    assert c.length(a) == 65 and c.length(b) == 64
    assert len(c.page_rows(0, [a])[0]) == 2 and len(c.page_rows(0, [b])[0]) == 1
    c.check_invariants()
    c.reserve([(b, 1)])            # crosses into its second page
    c.commit(b, 1)
    assert len(c.page_rows(1, [b])[0]) == 2
    with pytest.raises(CacheFull):
        c.reserve([(a, 64 * 2), (b, 64)])   # 6 pages in all; 4 held, 3 more asked
    c.check_invariants()
    assert len(c.page_rows(0, [a])[0]) == 2  # the failed reserve changed nothing
    held = set(c.page_rows(0, [a])[0])
    c.release(a)
    with pytest.raises(CacheError):
        c.release(a)
    d = c.acquire()
    assert d == a and c.length(d) == 0       # the slot is used again, empty
    c.reserve([(d, 128)])
    assert set(c.page_rows(0, [d])[0]) == held   # and so are its pages
    c.check_invariants()


def test_a_slot_number_means_the_same_sequence_only_while_the_counter_stands_still():
    """What a recorded decode step keeps on the device about its slots stays valid only as long as nobody was
    given or gave back a slot: the cache counts both, and nothing else moves the count."""
    c = _cache()
    n0 = c.ownership_changes
    a = c.acquire()
    assert c.ownership_changes == n0 + 1
    c.reserve([(a, 70)])
    c.commit(a, 70)
    c.length(a), c.page_rows(0, [a])
    assert c.ownership_changes == n0 + 1
    with pytest.raises(CacheFull):
        c.reserve([(a, 64 * 10)])
    assert c.ownership_changes == n0 + 1
    c.release(a)
    assert c.ownership_changes == n0 + 2
    with pytest.raises(CacheError):
        c.release(a)                       # a refused release is no change of owner
    assert c.ownership_changes == n0 + 2
    assert c.acquire() == a and c.ownership_changes == n0 + 3   # same number, another sequence


def test_random_walk_never_loses_or_doubles_a_page():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 16, max_slots=5)
    live = []
    for _ in range(2000):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            live.append(c.acquire())
        elif op < 0.45 and live:
            c.release(live.pop(rng.randrange(len(live))))
        elif live:
            s = rng.choice(live)
            n = rng.choice([1, 1, 1, 7, 64, 130])
            try:
                c.reserve([(s, n)])
                c.commit(s, n)
            except CacheFull:
                pass
        c.check_invariants()
        for g in c.paged_groups:
            assert g.pool.n_held == sum(pages_for(c.length(s)) for s in live)
    for s in live:
        c.release(s)
    assert all(g.pool.n_free == g.pool.n_pages for g in c.paged_groups) and c.slots.n_free == 5


def test_windowed_group_lets_go_of_pages_no_query_can_reach():
    needs = {0: KVCacheNeed(1, 16), 1: KVCacheNeed(1, 16, window=70)}
    c = SequenceCache(needs, max_tokens=64 * 32, max_slots=2, dtype=torch.float32, device="cpu", window_slack=64)
    full, win = (g for g in c.paged_groups)
    assert full.need.window is None and win.need.window == 70
    assert win.pool.n_pages == 2 * (pages_for(70 + 64) + 1) < full.pool.n_pages
    s = c.acquire()
    for _ in range(10):
        c.reserve([(s, 64)])
        c.commit(s, 64)
        c.check_invariants()
    rows_full, rows_win = c.page_rows(0, [s])[0], c.page_rows(1, [s])[0]
    assert len(rows_full) == 10 and all(p >= 0 for p in rows_full)
    # length 640: the next query (position 640) reads keys 571..640, i.e. from page 8 on
    assert rows_win[:8] == [-1] * 8 and all(p >= 0 for p in rows_win[8:])
    c.release(s)
    assert win.pool.n_free == win.pool.n_pages


def test_fixed_size_state_is_zeroed_when_a_slot_is_taken():
    needs = {0: KVCacheNeed(1, 16), 1: StateNeed((3, 4)), 2: StateNeed((3, 4)), 3: StateNeed((2,), torch.int32)}
    c = SequenceCache(needs, max_tokens=128, max_slots=3, dtype=torch.float32, device="cpu")
    assert len(c.slot_groups) == 2 and tuple(c.slot_groups[0].data.shape) == (2, 3, 3, 4)
    s = c.acquire()
    c.view(1).data[s] += 5.0
    c.view(3).data[s] += 2
    assert float(c.view(2).data[s].sum()) == 0.0   # entries do not share state
    c.release(s)
    s2 = c.acquire()
    assert s2 == s and float(c.view(1).data[s2].abs().sum()) == 0.0 and int(c.view(3).data[s2].sum()) == 0


def test_llama_has_no_fixed_state_but_the_cache_has_room_for_it():
    c = _cache()
    assert c.slot_groups == []
