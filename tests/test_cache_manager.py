"""Cache manager: pages, block tables, windows, slots (CPU).  No page is lost,
held twice or freed twice, under random orders of requests."""

import random

import pytest
from hypothesis import given, settings, strategies as st

from prism_b200.cache.manager import CacheManager, OutOfPages, OutOfSlots, PageAllocator, plan_groups
from prism_b200.parts.base import CacheNeed

FULL = CacheNeed("paged", 2, 16, None)
WIN = CacheNeed("paged", 2, 16, 20)
STATE = CacheNeed("state", state_shape=(4,))


def manager(needs, page_size=8, num_pages=12, max_seqs=4, max_seq_len=128):
    groups, where = plan_groups(needs, [None] * len(needs))
    return CacheManager(groups, page_size, num_pages, max_seqs, max_seq_len), groups, where


def test_groups_by_need_and_shared_planes():
    needs = [FULL, WIN, FULL, None, STATE, WIN]
    groups, where = plan_groups(needs, [None, None, None, 0, None, None])
    assert [g.need for g in groups] == [FULL, WIN, STATE]
    assert [g.entries for g in groups] == [[0, 2], [1, 5], [4]]
    assert where[3] == (0, 0, False)          # entry 3 reads entry 0's plane and does not own one
    assert where[2] == (0, 1, True) and where[4] == (2, 0, True)


def test_lifo_page_zero_first_and_reuse():
    a = PageAllocator(4)
    assert [a.alloc() for _ in range(3)] == [0, 1, 2]
    a.free(1)
    assert a.alloc() == 1 and a.alloc() == 3
    with pytest.raises(OutOfPages):
        a.alloc()
    with pytest.raises(AssertionError):
        a.free(5)
    a.free(0)
    with pytest.raises(AssertionError):
        a.free(0)                              # freed twice


def test_append_is_all_or_nothing_and_commit_advances():
    m, _, _ = manager([FULL], page_size=8, num_pages=3)
    m.add_request("a")
    assert m.pages_needed("a", 17) == [3] and m.can_append("a", 17)
    m.append("a", 17)
    m.commit("a", 17)
    assert m.length("a") == 17 and m.block_table_row("a", 0) == [0, 1, 2]
    m.add_request("b")
    assert not m.can_append("b", 1)
    with pytest.raises(OutOfPages):
        m.append("b", 1)
    m.check_invariants()
    assert m.num_free_pages(0) == 0
    m.append("a", 7)                            # fits in the last page
    m.commit("a", 7)
    assert not m.can_append("a", 1)
    m.free_request("a")
    assert m.num_free_pages(0) == 3
    m.append("b", 1)
    m.check_invariants()


def test_window_pages_are_given_back_as_the_window_passes():
    m, _, _ = manager([FULL, WIN], page_size=8, num_pages=16, max_seq_len=200)
    m.add_request("a")
    m.append("a", 50)
    m.commit("a", 50)
    # next query at 50 sees keys 31..50 in the window group: pages 0..2 (keys 0..23) are free again
    assert m.block_table_row("a", 1)[:4] == [-1, -1, -1, 3]
    assert m.block_table_row("a", 0) == list(range(7))
    assert m.num_free_pages(1) == 16 - 4 and m.num_free_pages(0) == 16 - 7
    for _ in range(30):
        m.append("a", 1)
        m.commit("a", 1)
        m.check_invariants()
    live = [p for p in m.block_table_row("a", 1) if p >= 0]
    assert len(live) <= 20 // 8 + 2            # a window of 20 never holds more than 4 pages of 8
    m.free_request("a")
    assert m.num_free_pages(1) == 16 and m.num_free_pages(0) == 16


def test_slots():
    m, _, _ = manager([STATE], max_seqs=2)
    assert m.add_request("a") == 0 and m.add_request("b") == 1
    assert m.drain_fresh_slots() == [0, 1] and m.drain_fresh_slots() == []
    with pytest.raises(OutOfSlots):
        m.add_request("c")
    with pytest.raises(KeyError):
        m.add_request("a")
    m.free_request("a")
    assert m.add_request("c") == 0 and m.drain_fresh_slots() == [0]
    m.append("c", 5)                            # a state-only model needs no pages
    m.commit("c", 5)
    m.check_invariants()


def test_sequence_limit():
    m, _, _ = manager([FULL], num_pages=100, max_seq_len=20)
    m.add_request("a")
    assert not m.can_append("a", 21)
    with pytest.raises(ValueError):
        m.append("a", 21)


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 10 ** 6), st.integers(1, 3), st.sampled_from([1, 4, 8]), st.integers(3, 20))
def test_random_orders_keep_the_invariants(seed, n_groups, page_size, num_pages):
    rng = random.Random(seed)
    needs = [[FULL], [FULL, WIN], [WIN, STATE, FULL]][n_groups - 1]
    m, groups, _ = manager(needs, page_size=page_size, num_pages=num_pages, max_seqs=3, max_seq_len=64)
    live, next_id = [], 0
    for _ in range(200):
        op = rng.random()
        if op < 0.25 and len(live) < 3:
            m.add_request(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(live)
            n = rng.randint(1, 9)
            if m.can_append(r, n):
                before = [m.num_free_pages(g.index) for g in groups if g.kind == "paged"]
                m.append(r, n)
                m.commit(r, n)
            else:
                before = [m.num_free_pages(g.index) for g in groups if g.kind == "paged"]
                with pytest.raises((OutOfPages, ValueError)):
                    m.append(r, n)
                assert before == [m.num_free_pages(g.index) for g in groups if g.kind == "paged"]
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.free_request(r)
        m.check_invariants()
        for r in live:                          # every position a later query can see has a page
            L = m.length(r)
            for g in groups:
                if g.kind != "paged":
                    continue
                lo = max(0, L - g.need.window + 1) if g.need.window else 0
                row = m.block_table_row(r, g.index)
                assert all(row[p // page_size] >= 0 for p in range(lo, L))
    m.free_all()
    m.check_invariants()
    assert all(m.num_free_pages(g.index) == num_pages for g in groups if g.kind == "paged")


def test_pool_sizes_per_group():
    """A windowed group gets the pages its window and one portion need for every request slot, not the
    pool of a group that keeps every key; a budget pays the windowed groups first."""
    from prism_b200.cache.manager import pool_sizes
    groups, _ = plan_groups([FULL, WIN, FULL, STATE, WIN], [None] * 5)
    # explicit size: full groups get it, the windowed group ceil((20 + 16) / 8) + 1 = 6 pages for each of 4 slots
    assert pool_sizes(groups, 8, 2, 128, 4, 16, num_pages=40) == [40, 24, 0]
    assert pool_sizes(groups, 8, 2, 128, 4, 16, num_pages=10) == [10, 10, 0]        # never more than the others
    # budget: bytes of a page = 2 (k, v) * planes * P * nkv * hd * element bytes
    full_page = win_page = 2 * 2 * 8 * 2 * 16 * 2
    budget = 24 * win_page + 30 * full_page + 5
    assert pool_sizes(groups, 8, 2, 128, 4, 16, budget_bytes=budget) == [30, 24, 0]
    assert pool_sizes(groups, 8, 2, 128, 4, 16, budget_bytes=1e12) == [64, 24, 0]      # cap: 4 requests of 128 tokens
    assert pool_sizes(groups, 8, 2, 128, 4, 16, budget_bytes=0) == [16, 16, 0]         # floor (engine/scheduler.py:103)
    # a windowed model runs any workload in that pool: portions of 16 tokens, 4 requests, long sequences
    m = CacheManager(groups, 8, pool_sizes(groups, 8, 2, 128, 4, 16, num_pages=64), 4, 128)
    for r in range(4):
        m.add_request(r)
    for _ in range(8):
        for r in range(4):
            assert m.can_append(r, 16)
            m.append(r, 16)
        for r in range(4):
            m.commit(r, 16)
        m.check_invariants()
