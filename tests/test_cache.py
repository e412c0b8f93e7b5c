"""The cache's bookkeeping: no slot or page lost, held twice or freed twice; groups with
different needs have storage of their own; window groups give pages back."""
import random

import numpy as np
import pytest

from oracle_engine_b200.cache.kv_cache import KVCache, pages_for
from oracle_engine_b200.cache.slots import CacheFull, PagePool, SlotAllocator
from oracle_engine_b200.parts.spec import CacheNeed, attention_cache_need

FULL = attention_cache_need(2, 16)
WIN = attention_cache_need(2, 16, 100)


def test_slot_allocator():
    a = SlotAllocator(3)
    s = [a.alloc(), a.alloc(), a.alloc()]
    assert sorted(s) == [0, 1, 2]
    with pytest.raises(CacheFull):
        a.alloc()
    a.free(1)
    with pytest.raises(ValueError, match="freed twice"):
        a.free(1)
    with pytest.raises(ValueError):
        a.free(7)
    assert a.alloc() == 1            # freed slots are used again
    a.check()


def test_page_pool():
    p = PagePool(2)
    x, y = p.alloc(), p.alloc()
    with pytest.raises(CacheFull):
        p.alloc()
    p.release(x)
    with pytest.raises(ValueError, match="twice"):
        p.release(x)
    assert p.alloc() == x and y != x
    p.check()


def test_groups_have_their_own_storage():
    needs = [FULL, WIN, FULL, None, attention_cache_need(1, 32), WIN]
    c = KVCache(needs, max_tokens=640, max_seq_len=512, allocate=False, window_pool_tokens=256)
    assert [g.need for g in c.groups] == [FULL, WIN, attention_cache_need(1, 32)]
    assert [g.entries for g in c.groups] == [[0, 2], [1, 5], [4]]
    assert c.entry_group[2] == (0, 1) and 3 not in c.entry_group
    assert [g.pool.n for g in c.groups] == [10, 4, 10]
    assert c.max_pages_per_seq == 8


def test_reserve_free_and_reuse():
    c = KVCache([FULL, FULL], max_tokens=256, max_seq_len=256, allocate=False)
    a, b = c.alloc_slot(), c.alloc_slot()
    assert c.reserve(a, 65) and not c.reserve(a, 100)       # two pages, then nothing new
    c.commit(a, 100)
    c.reserve(b, 128)
    c.commit(b, 128)
    assert c.groups[0].pool.n_free == 0
    with pytest.raises(CacheFull):
        c.reserve(a, 129)
    assert (c.groups[0].tables[a] >= 0).sum() == 2         # a failed reserve changes nothing
    c.check()
    pages_b = set(c.groups[0].tables[b][:2].tolist())
    c.free_slot(b)
    with pytest.raises(ValueError, match="freed twice"):
        c.free_slot(b)
    assert c.length(b) == 0
    d = c.alloc_slot()
    assert d == b
    c.reserve(d, 70)
    assert set(c.groups[0].tables[d][:2].tolist()) == pages_b           # pages are used again
    with pytest.raises(CacheFull, match="allows 256"):
        c.reserve(d, 257)
    c.check()


def test_window_group_releases_pages():
    c = KVCache([FULL, WIN], max_tokens=1024, max_seq_len=1024, allocate=False)
    s = c.alloc_slot()
    c.reserve(s, 300)
    c.commit(s, 300)
    full, win = c.groups
    assert (win.tables[s] >= 0).sum() == pages_for(300)
    c.reserve(s, 301)                  # first new query at 300 reads keys >= 201: page 3 on
    c.commit(s, 301)
    assert win.tables[s][:3].tolist() == [-1, -1, -1] and (win.tables[s][3:5] >= 0).all()
    assert (full.tables[s][:5] >= 0).all()
    c.check()
    c.free_slot(s)
    assert win.pool.n_free == win.pool.n and full.pool.n_free == full.pool.n
    c.check()


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    c = KVCache([FULL, WIN, FULL], max_tokens=2048, max_seq_len=700, allocate=False, window_pool_tokens=1024)
    live = {}
    for _ in range(2000):
        r = rng.random()
        if r < 0.3 and c.slots.n_free:
            live[c.alloc_slot()] = 0
        elif r < 0.5 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 1, 17, 64, 130])
            try:
                c.reserve(s, n)
                c.commit(s, n)
                live[s] = n
            except CacheFull:
                pass
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
            assert (c.groups[0].tables[s][:pages_for(n)] >= 0).all()
    for s in list(live):
        c.free_slot(s)
    c.check()
    assert all(g.pool.n_free == g.pool.n for g in c.groups)


def test_tables_for_padding():
    c = KVCache([FULL], max_tokens=256, max_seq_len=256, allocate=False)
    s = c.alloc_slot()
    c.reserve(s, 10)
    t = c.tables_for(0, np.array([s, -1], dtype=np.int32))
    assert t.shape == (2, 4) and t[0, 0] >= 0 and (t[1] == -1).all()
