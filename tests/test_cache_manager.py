"""The page pools and the cache manager (host code, no GPU)."""

from __future__ import annotations

import random

import pytest

from llm_inference_b200.csrc.host_module import host


@pytest.fixture(scope="module")
def h():
    return host()


def test_pool_lowest_free_first_and_reservations(h):
    pool = h.PagePool(4)
    assert [pool.allocate(reserved=False) for _ in range(3)] == [0, 1, 2]
    pool.release(1)
    assert pool.allocate(reserved=False) == 1  # the lowest free id again
    assert pool.reserve(1) and not pool.reserve(1)
    with pytest.raises(RuntimeError, match="exhausted"):
        pool.allocate(reserved=False)  # the last free page is promised
    assert pool.allocate(reserved=True) == 3
    with pytest.raises(RuntimeError, match="isn't allocated"):
        pool.release(7)
    pool.release(2)
    with pytest.raises(RuntimeError, match="isn't allocated"):
        pool.release(2)  # freed twice
    with pytest.raises(RuntimeError, match="more pages than were reserved"):
        pool.unreserve(1)
    pool.retain(0)
    pool.release(0)
    assert pool.used == 3 and pool.high_water == 4
    pool.release(0)
    assert pool.used == 2


def manager(h, pages=8, window_pages=6, page=4, window=6, slots=0, step=4):
    groups = [h.GroupSpec("full", pages, 0)]
    if window:
        groups.append(h.GroupSpec("window", window_pages, window))
    return h.CacheManager(page, groups, slots, step)


def test_page_edges_and_reserve_before_start(h):
    m = manager(h, window=0)
    assert m.needs(15) == [4] and m.needs(16) == [4] and m.needs(17) == [5]
    assert m.admit(1, 17) and m.stats()["kv_pools"]["full"]["reserved_pages"] == 5
    assert not m.admit(2, 16)  # only 3 pages are not promised
    assert m.stats()["allocation_failures"] == 1
    assert m.admit(2, 12)
    m.ensure(1, 4)
    assert m.table(1, 0) == [0]
    m.ensure(1, 5)
    assert m.table(1, 0) == [0, 1]
    m.ensure(2, 1)
    assert m.table(2, 0) == [2]
    m.ensure(1, 17)
    assert m.table(1, 0) == [0, 1, 3, 4, 5]
    with pytest.raises(RuntimeError, match="exceeded its K/V reservation"):
        m.ensure(1, 21)
    m.check_invariants()
    m.release(1)
    m.ensure(2, 12)
    assert m.table(2, 0) == [2, 0, 1]  # request 1's pages are used again
    m.release(2)
    m.release(2)  # releasing twice is harmless
    stats = m.stats()["kv_pools"]["full"]
    assert stats["used_pages"] == 0 and stats["reserved_pages"] == 0
    m.check_invariants()


def test_window_group_gives_pages_back_and_reuses_them(h):
    m = manager(h, pages=16, window_pages=6, page=4, window=6, step=4)
    assert m.needs(64) == [16, 4]  # ceil((6 + 4) / 4) + 1
    assert m.admit(1, 64)
    peak = 0
    for length in range(1, 65):
        m.ensure(1, length)
        m.advance(1, length)
        m.check_invariants()
        peak = max(peak, m.stats()["kv_pools"]["window"]["used_pages"])
        table = m.table(1, 1)
        first_live = max(0, length - 6 + 1) // 4
        assert all(p == -1 for p in table[:first_live]) and all(p >= 0 for p in table[first_live:])
    assert peak <= 3 and m.stats()["kv_pools"]["full"]["used_pages"] == 16
    assert max(m.table(1, 1)) <= 3  # trimmed pages came back under the lowest ids
    m.release(1)
    m.check_invariants()
    assert m.stats()["kv_pools"]["window"]["reserved_pages"] == 0


def test_open_without_reservation_runs_out_loudly(h):
    m = manager(h, pages=2, window=0)
    m.open(1)
    m.ensure(1, 8)
    m.open(2)
    with pytest.raises(RuntimeError, match="exhausted"):
        m.ensure(2, 1)
    m.release(1)
    m.ensure(2, 1)
    assert m.table(2, 0) == [0]


def test_state_slots(h):
    m = manager(h, window=0, slots=2)
    assert m.admit(1, 4) and m.admit(2, 4)
    assert {m.slot(1), m.slot(2)} == {0, 1}
    assert sorted(m.take_slots_to_clear()) == [0, 1] and m.take_slots_to_clear() == []
    assert not m.admit(3, 4)  # pages are free, slots are not
    m.release(1)
    assert m.admit(3, 4) and m.take_slots_to_clear() == [m.slot(3)]
    m.check_invariants()


def test_random_traffic_conserves_pages(h):
    rng = random.Random(7)
    m = manager(h, pages=24, window_pages=12, page=4, window=10, slots=5, step=6)
    live: dict[int, list[int]] = {}  # id -> [length, budget]
    next_id = 1
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            budget = rng.randint(1, 40)
            if m.admit(next_id, budget):
                live[next_id] = [0, budget]
            next_id += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            length, budget = live[rid]
            grow = min(rng.randint(1, 6), budget - length)
            if grow:
                m.ensure(rid, length + grow)
                m.advance(rid, length + grow)
                live[rid][0] += grow
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        stats = m.stats()
        assert stats["requests"] == len(live)
        for pool in stats["kv_pools"].values():
            assert pool["used_pages"] + pool["free_pages"] == pool["capacity_pages"]
            assert pool["reserved_pages"] <= pool["free_pages"]
    for rid in list(live):
        m.release(rid)
    stats = m.stats()
    assert all(p["used_pages"] == 0 and p["reserved_pages"] == 0 for p in stats["kv_pools"].values())
    assert stats["free_state_slots"] == 5
