"""The cache manager on the CPU: pages, block tables, windows, state slots; no page lost, held twice or freed
twice under random orders of requests."""
from __future__ import annotations

import random

import pytest

from cuinfer_b200.cache import CacheError, CacheGroupSpec, CacheManager, PagePool, SlotPool, group_runs
from cuinfer_b200.parts import PagedCacheNeed


def full_group(runs=(0, 1)):
    return CacheGroupSpec(tuple(runs), 2, 16, None)


def test_page_pool_fifo_and_double_free():
    pool = PagePool(4)
    a = pool.take(3)
    assert a == [0, 1, 2] and pool.num_free == 1
    assert pool.take(2) is None and pool.num_free == 1          # all or nothing
    pool.give_back([1])
    assert pool.take(2) == [3, 1]                               # freed pages go to the tail
    with pytest.raises(CacheError, match="twice"):
        pool.give_back([0, 0])
    with pytest.raises(CacheError):
        pool.give_back([9])
    pool.check()


def test_slot_pool():
    slots = SlotPool(2)
    assert slots.take() == 0 and slots.take() == 1 and slots.take() is None
    slots.give_back(0)
    with pytest.raises(CacheError):
        slots.give_back(0)
    assert slots.take() == 0


def test_allocation_tables_and_slot_mapping():
    mgr = CacheManager([full_group()], page_size=4, num_pages=6, max_requests=3)
    assert mgr.admit("a") == 0
    with pytest.raises(CacheError, match="already"):
        mgr.admit("a")
    assert mgr.pages_needed("a", 5) == [2]
    assert mgr.allocate("a", 5) and mgr.block_table("a") == [0, 1]
    assert mgr.slot_mapping("a", 0, 0, 5) == [0, 1, 2, 3, 4]
    mgr.commit("a", 5)
    assert mgr.allocate("a", 3) and mgr.block_table("a") == [0, 1]     # 8 tokens still fit two pages
    mgr.commit("a", 3)
    assert mgr.allocate("a", 1) and mgr.block_table("a") == [0, 1, 2]
    assert mgr.slot_mapping("a", 0, 8, 1) == [8]
    mgr.commit("a", 1)
    assert mgr.admit("b") == 1
    assert not mgr.allocate("b", 13)                                    # needs 4 pages, 3 free: nothing taken
    assert mgr.num_free_pages() == 3 and mgr.block_table("b") == []
    assert mgr.allocate("b", 12)
    with pytest.raises(CacheError, match="do not fit"):
        mgr.commit("b", 13)
    mgr.release("a")
    assert mgr.num_free_pages() == 3
    assert mgr.admit("c") == 0                                          # a's slot is used again
    assert mgr.allocate("c", 4) and mgr.block_table("c") == [0]         # and its first page
    with pytest.raises(CacheError):
        mgr.release("a")
    mgr.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    groups = [CacheGroupSpec((0,), 2, 16, None), CacheGroupSpec((1,), 2, 16, 6)]
    mgr = CacheManager(groups, page_size=4, num_pages=[8, 4], max_requests=2)
    mgr.admit("a")
    held_peak = 0
    for step in range(24):
        assert mgr.allocate("a", 1), f"window group ran out at token {step}"
        mgr.commit("a", 1)
        held = sum(1 for p in mgr.block_table("a", 1) if p >= 0)
        held_peak = max(held_peak, held)
        total = step + 1
        first_needed = max(0, total - 6 + 1)
        # every page the next query can still see is held; every page before is given back
        for idx, page in enumerate(mgr.block_table("a", 1)):
            assert (page >= 0) == (idx >= first_needed // 4), (step, idx, mgr.block_table("a", 1))
        mgr.check()
    assert held_peak <= 3 and len(mgr.block_table("a", 0)) == 6 and all(p >= 0 for p in mgr.block_table("a", 0))
    # the second group is the scarce one: an allocation that fits group 0 but not group 1 takes nothing
    mgr.admit("b")
    free0 = mgr.num_free_pages(0)
    assert not mgr.allocate("b", 13)
    assert mgr.num_free_pages(0) == free0
    mgr.release("a")
    mgr.release("b")
    assert mgr.num_free_pages(0) == 8 and mgr.num_free_pages(1) == 4


def test_group_runs_by_need():
    needs = {0: PagedCacheNeed(2, 16), 1: PagedCacheNeed(2, 16, 128), 2: PagedCacheNeed(2, 16), 4: PagedCacheNeed(4, 16)}
    groups = group_runs(needs)
    assert [g.runs for g in groups] == [(0, 2), (1,), (4,)]
    assert [g.window for g in groups] == [None, 128, None]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    groups = [CacheGroupSpec((0, 1), 2, 16, None), CacheGroupSpec((2,), 1, 32, 10)]
    mgr = CacheManager(groups, page_size=4, num_pages=[rng.randint(6, 20), rng.randint(5, 12)], max_requests=4)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 6:
            rid = f"r{next_id}"
            next_id += 1
            slot = mgr.admit(rid)
            if slot is None:
                assert len(live) >= 4
            else:
                live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 9, 17])
            before = [mgr.num_free_pages(g) for g in range(2)]
            if mgr.allocate(rid, n):
                positions = mgr.slot_mapping(rid, 0, live[rid], n)
                assert len(set(positions)) == n
                mgr.commit(rid, n)
                live[rid] += n
                assert mgr.num_tokens(rid) == live[rid]
            else:
                assert [mgr.num_free_pages(g) for g in range(2)] == before
        elif live:
            rid = rng.choice(list(live))
            mgr.release(rid)
            del live[rid]
        mgr.check()
        # no page is in two live tables of a group
        for g in range(2):
            pages = [p for rid in live for p in mgr.block_table(rid, g) if p >= 0]
            assert len(pages) == len(set(pages))
    for rid in list(live):
        mgr.release(rid)
    mgr.check()
    assert mgr.num_free_pages(0) == mgr.pools[0].num_pages and mgr.num_free_pages(1) == mgr.pools[1].num_pages
    assert mgr.slots.num_free == 4
