"""The cache manager: no page lost, held twice or freed twice, under random
orders of requests; first-in first-out reuse; windows give pages back; state
slots.  (Reference behaviours: tests/block_manager_test.cc:16-50.)"""
import random

import pytest
import torch

from chibillm_b200.cache import (CacheError, CacheManager, CacheStorage, GroupLayout, PagePool, plan_cache,
                                 first_needed_block, pages_for)
from chibillm_b200.parts import FixedStateNeed, PagedKVNeed, Runtime


def manager(pages=8, page_size=4, window=None, max_requests=4):
    groups = [GroupLayout("full", 2, 16, None, page_size, pages, 2)]
    if window:
        groups.append(GroupLayout("win", 2, 16, window, page_size, pages, 1))
    return CacheManager(groups, max_requests)


def test_growth_at_page_boundaries():
    m = manager()
    m.admit(1)
    m.reserve(1, 1)
    assert m.get(1).tables["full"] == [0]
    m.reserve(1, 4)
    assert m.get(1).tables["full"] == [0]
    m.reserve(1, 5)
    assert m.get(1).tables["full"] == [0, 1]
    m.reserve(1, 3)                              # never shrinks
    assert m.get(1).tables["full"] == [0, 1]
    with pytest.raises(CacheError) as e:
        m.reserve(1, 0)
    assert e.value.code == "invalid_reservation"
    with pytest.raises(CacheError) as e:
        m.reserve(2, 1)
    assert e.value.code == "unknown_request"


def test_fifo_reuse_order():
    m = manager(pages=4)
    m.admit("a"); m.reserve("a", 8)              # pages 0, 1
    m.admit("b"); m.reserve("b", 4)              # page 2
    m.release("a")                               # free list: 3, 0, 1
    m.admit("c"); m.reserve("c", 12)
    assert m.get("c").tables["full"] == [3, 0, 1]
    m.release("a")                               # releasing twice is harmless
    m.check_invariants()


def test_failed_reservation_changes_nothing():
    m = manager(pages=3, window=6)
    m.admit(1); m.reserve(1, 8)
    m.admit(2)
    before = (m.free_pages("full"), m.free_pages("win"), dict(m.get(2).tables))
    with pytest.raises(CacheError) as e:
        m.reserve(2, 8)
    assert e.value.code == "capacity_exhausted"
    assert (m.free_pages("full"), m.free_pages("win"), dict(m.get(2).tables)) == before
    m.check_invariants()


def test_double_free_and_foreign_pages_are_refused():
    pool = PagePool(4)
    a = pool.take(2)
    pool.give(a)
    with pytest.raises(CacheError):
        pool.give(a)
    with pytest.raises(CacheError):
        pool.give([9])
    with pytest.raises(CacheError):
        pool.take(5)


def test_window_gives_pages_back():
    assert first_needed_block(0, 6, 4) == 0
    assert first_needed_block(9, 6, 4) == 1      # a query at 9 sees 4..9 -> block 1 on
    assert first_needed_block(10, 6, 4) == 1
    assert first_needed_block(13, 6, 4) == 2
    m = manager(pages=16, window=6)
    m.admit(1)
    m.reserve(1, 20)
    assert len([p for p in m.get(1).tables["win"] if p >= 0]) == 5
    m.commit(1, 20)                              # next query at 20 sees 15..20 -> blocks 3, 4
    assert m.get(1).tables["win"] == [-1, -1, -1, 3, 4]
    assert m.get(1).tables["full"] == [0, 1, 2, 3, 4]
    assert m.free_pages("win") == 14 and m.free_pages("full") == 11
    for length in range(21, 40):
        m.reserve(1, length)
        m.commit(1, length)
        held = [p for p in m.get(1).tables["win"] if p >= 0]
        assert len(held) <= pages_for(6, 4) + 1
        m.check_invariants()
    with pytest.raises(CacheError):
        m.commit(1, 100)                         # beyond the reservation
    m.release(1)
    assert m.free_pages("win") == 16 and m.free_pages("full") == 16


def test_state_slots():
    m = manager(max_requests=2)
    a, b = m.admit("a"), m.admit("b")
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(CacheError) as e:
        m.admit("c")
    assert e.value.code == "capacity_exhausted"
    with pytest.raises(CacheError) as e:
        m.admit("a")
    assert e.value.code == "duplicate_request"
    m.release("a")
    assert m.admit("c").state_slot == a.state_slot
    m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = manager(pages=24, page_size=4, window=10, max_requests=5)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 5, 9, 17])
            try:
                m.reserve(rid, live[rid] + grow)
            except CacheError as e:
                assert e.code == "capacity_exhausted"
            else:
                if rng.random() < 0.9:           # sometimes a step is aborted: reserved, not committed
                    live[rid] += grow
                    m.commit(rid, live[rid])
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            rc = m.get(rid)
            assert rc.length == n
            # every position a later query can see has a page
            full = rc.tables["full"]
            assert all(p >= 0 for p in full[:pages_for(n, 4)])
            win = rc.tables["win"]
            for blk in range(first_needed_block(n, 10, 4), pages_for(n, 4)):
                assert win[blk] >= 0
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.free_pages("full") == 24 and m.free_pages("win") == 24 and m.slots.free_count == 5


def test_plan_groups_by_need_and_shares_caches():
    full = PagedKVNeed(2, 16, None)
    win = PagedKVNeed(2, 16, 32)
    state = FixedStateNeed((("h", (8,), torch.float32),))
    plan = plan_cache([full, win, full, state, full, None], [None, None, None, None, 0, None],
                      page_size=8, pool_tokens=60)
    names = {g.name: g for g in plan.groups}
    assert set(names) == {"kv2x16", "kv2x16w32"}
    assert names["kv2x16"].num_entries == 2 and names["kv2x16w32"].num_entries == 1
    assert names["kv2x16"].num_pages == 8                       # 60 tokens -> 8 pages of 8
    assert plan.steps[0] == ("paged", "kv2x16", 0, True)
    assert plan.steps[2] == ("paged", "kv2x16", 1, True)
    assert plan.steps[4] == ("paged", "kv2x16", 0, False)       # reads step 0's cache
    assert plan.steps[3][0] == "state" and plan.steps[5] is None
    with pytest.raises(CacheError):
        plan_cache([full, full], [None, 5], 8, 64)
    with pytest.raises(CacheError):
        plan_cache([state, full], [None, 0], 8, 64)
    rt = Runtime(torch.device("cpu"), torch.float32, None)
    storage = CacheStorage(plan, rt, num_slots=3)
    assert storage.keys["kv2x16"].shape == (2, 8, 2, 8, 16)
    assert storage.views[4].keys.data_ptr() == storage.views[0].keys.data_ptr() and not storage.views[4].writes
    assert storage.views[3].arrays["h"].shape == (3, 8)
    storage.views[3].arrays["h"][1] = 5.0
    storage.zero_state_slot(1)
    assert float(storage.views[3].arrays["h"].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(4))
def test_device_mirror_follows_the_tables(seed):
    """The drained updates, applied in any order (the device applies them in
    parallel), keep a mirror [slot][block] equal to the host tables of the live
    requests -- also when a slot passes from one request to the next."""
    rng = random.Random(100 + seed)
    m = manager(pages=24, page_size=4, window=10, max_requests=3)
    mirror = {g: {} for g in m.groups}
    live = {}
    next_id = 0
    for step in range(400):
        r = rng.random()
        if r < 0.3 and len(live) < 3:
            m.admit(next_id); live[next_id] = 0; next_id += 1
        elif r < 0.8 and live:
            rid = rng.choice(list(live))
            grow = rng.choice([1, 1, 3, 9, 20])
            try:
                m.reserve(rid, live[rid] + grow)
                live[rid] += grow
                m.commit(rid, live[rid])
            except CacheError:
                pass
        elif live:
            rid = rng.choice(list(live)); m.release(rid); del live[rid]
        if rng.random() < 0.5:          # a step happens: updates travel to the device
            for g in m.groups:
                ups = m.drain_updates(g)
                assert len({(row, idx) for row, idx, _ in ups}) == len(ups)
                rng.shuffle(ups)
                for row, idx, page in ups:
                    mirror[g][(row, idx)] = page
                for rid in live:
                    rc = m.get(rid)
                    for idx, page in enumerate(rc.tables[g]):
                        assert mirror[g].get((rc.state_slot, idx), -1) == page


def test_a_reader_of_another_steps_cache_must_share_its_window():
    """A run step that reads another step's cache lives by the owner's window:
    pages behind it are given back.  A reader with another window is refused when
    the cache is planned, not in the middle of a generation."""
    from chibillm_b200.cache.manager import CacheError
    from chibillm_b200.cache.storage import plan_cache
    from chibillm_b200.parts import PagedKVNeed
    owner = PagedKVNeed(2, 16, 24)
    plan = plan_cache([owner, PagedKVNeed(2, 16, 24)], [None, 0], 8, 256)
    assert plan.steps[1][3] is False and len(plan.groups) == 1
    for reader in (PagedKVNeed(2, 16, None), PagedKVNeed(2, 16, 48), PagedKVNeed(2, 16, 8)):
        with pytest.raises(CacheError) as e:
            plan_cache([owner, reader], [None, 0], 8, 256)
        assert "windows differ" in str(e.value)


def test_held_commits_settle_and_roll_back():
    from chibillm_b200.cache.manager import CacheError, CacheManager, GroupLayout
    m = CacheManager([GroupLayout("w", 1, 16, 10, 4, 16, 1, 0), GroupLayout("all", 1, 16, None, 4, 16, 1, 0)], 2)
    m.admit("a")
    m.reserve("a", 12)
    m.commit_many(["a"], [12])
    free = m.free_pages("w")
    m.reserve("a", 30)
    m.commit_many(["a"], [30], hold=True)
    assert m.length("a") == 30 and m.free_pages("w") == free - 5, "a held commit gives nothing back"
    m.rollback_many(["a"], [12])
    assert m.length("a") == 12
    m.commit_many(["a"], [30], hold=True)
    m.settle_many(["a"])
    assert m.free_pages("w") > free - 5
    with pytest.raises(CacheError):
        m.rollback_many(["a"], [12])            # settled: the pages behind the window are gone
    m.check_invariants()
    m.release("a")
    assert m.free_pages("w") == 16 and m.free_pages("all") == 16
