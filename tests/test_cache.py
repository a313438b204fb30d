"""The cache's bookkeeping: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from llmplayer_b200.cache import PAGE_SIZE, FreeList, KVRequest, PageMap, SequenceCache, StateRequest
from llmplayer_b200.errors import CacheError, CacheFull


def test_free_list_hands_out_each_id_once():
    fl = FreeList(4, "slot")
    got = [fl.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and fl.num_free == 0
    with pytest.raises(CacheFull):
        fl.take()
    fl.give_back(2)
    with pytest.raises(CacheError, match="freed twice"):
        fl.give_back(2)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back(9)
    assert fl.take() == 2


def test_page_map_grows_by_pages_and_gives_all_back():
    pm = PageMap(6)
    pm.open(0)
    pm.open(1)
    pm.extend(0, 1)
    assert len(pm.table(0)) == 1
    pm.extend(0, PAGE_SIZE)
    assert len(pm.table(0)) == 1
    pm.extend(0, PAGE_SIZE + 1)
    assert len(pm.table(0)) == 2
    pm.extend(1, 3 * PAGE_SIZE)
    assert pm.pool.num_free == 1
    with pytest.raises(CacheFull):
        pm.extend(0, 4 * PAGE_SIZE)
    assert len(pm.table(0)) == 2 and pm.pool.num_free == 1          # all or nothing
    assert len(set(pm.table(0)) | set(pm.table(1))) == 5            # no page held twice
    pm.close(0)
    pm.close(1)
    assert pm.pool.num_free == 6
    with pytest.raises(KeyError):
        pm.close(0)


def test_window_gives_back_pages_no_query_can_reach():
    pm = PageMap(8, window=70)
    pm.open(0)
    pm.extend(0, 200)
    pm.trim(0, 200)            # next query at 200 sees keys 131..200: blocks 0 and 1 (positions < 128) are free
    assert pm.table(0)[:2] == [-1, -1] and all(p >= 0 for p in pm.table(0)[2:])
    assert pm.pool.num_free == 8 - 2
    pm.extend(0, 262)
    pm.trim(0, 262)
    assert pm.table(0)[2] == -1 and pm.table(0)[3] >= 0
    pm.close(0)
    assert pm.pool.num_free == 8


def make_cache(max_tokens=512, max_slots=4):
    reqs = [KVRequest(2, 16), KVRequest(2, 16), KVRequest(2, 16, window=64), StateRequest((3,)), None]
    return SequenceCache(reqs, max_tokens=max_tokens, max_slots=max_slots, kv_dtype=torch.float32, device="cpu")


def test_groups_have_storage_of_their_own():
    c = make_cache()
    assert len(c.groups) == 2
    full, windowed = c.groups
    assert full.storage.shape == (2, 8, 2, 2, PAGE_SIZE, 16) and windowed.storage.shape[0] == 1
    assert c.view(0).pages.data_ptr() != c.view(1).pages.data_ptr()
    assert c.view(0).group_index == c.view(1).group_index != c.view(2).group_index
    assert c.view(3).rows.shape == (4, 3) and c.view(4) is None


def test_slots_lengths_and_reuse():
    c = make_cache()
    a, b = c.acquire(), c.acquire()
    c.reserve([a, b], [5, 70])
    c.commit([a, b], [5, 70])
    assert (c.length(a), c.length(b)) == (5, 70)
    assert c.free_pages() == [8 - 3, 8 - 3]
    with pytest.raises(CacheError, match="twice"):
        c.reserve([a, a], [1, 1])
    c.release(a)
    with pytest.raises(CacheError):
        c.release(a)
    with pytest.raises(CacheError):
        c.length(a)
    again = c.acquire()
    assert again == a and c.length(again) == 0          # the slot is used again, from length 0
    c.release(again)
    c.release(b)
    assert c.free_pages() == [8, 8] and c.slots.num_free == 4


def test_reserve_is_all_or_nothing_across_groups():
    c = make_cache(max_tokens=256)       # 4 pages per group
    a, b = c.acquire(), c.acquire()
    c.reserve([a], [130])                # 3 pages
    c.commit([a], [130])
    before = c.free_pages()
    with pytest.raises(CacheFull):
        c.reserve([a, b], [1, 100])      # b would need 2 pages, 1 is free
    assert c.free_pages() == before


def test_state_rows_are_zeroed_on_acquire():
    c = make_cache()
    a = c.acquire()
    c.view(3).rows[a] += 5.0
    c.release(a)
    assert c.acquire() == a and float(c.view(3).rows[a].abs().sum()) == 0.0


def test_no_slot_or_page_is_lost_under_churn():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 24, max_slots=6)
    held = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and c.slots.num_free:
            held[c.acquire()] = 0
        elif op < 0.5 and held:
            s = rng.choice(list(held))
            c.release(s)
            del held[s]
        elif held:
            s = rng.choice(list(held))
            n = rng.randint(1, 90)
            try:
                c.reserve([s], [n])
            except CacheFull:
                continue
            c.commit([s], [n])
            held[s] += n
        for g in c.groups:
            live = [p for s in held for p in g.pages.table(s) if p >= 0]
            assert len(live) == len(set(live)), "a page is held twice"
            assert len(live) + g.pages.pool.num_free == g.pages.pool.count, "a page was lost"
        assert all(c.length(s) == n for s, n in held.items())
        assert c.slots.num_held == len(held)
    for s in list(held):
        c.release(s)
    assert all(g.pages.pool.num_free == g.pages.pool.count for g in c.groups) and c.slots.num_free == 6
