"""The cache manager: no page lost, held twice or freed twice, under random orders of requests; groups with and
without a window; state slots."""
import numpy as np
import pytest
import torch

from infer_b200.cache import CacheError, CacheManager, PagePool
from infer_b200.parts.base import PagedKVNeed, StateNeed


def _manager(n_pages=16, page=4, slots=4, window=None, with_state=False):
    needs = {0: PagedKVNeed(2, 8, None), 1: PagedKVNeed(2, 8, None)}
    if window:
        needs[2] = PagedKVNeed(2, 8, window)
    if with_state:
        needs[3] = StateNeed({"s": ((3,), torch.float32)})
    return CacheManager(needs, n_pages, page, slots)


def test_pool_hands_out_and_reuses():
    p = PagePool(3)
    assert [p.alloc(), p.alloc(), p.alloc()] == [0, 1, 2] and p.alloc() is None
    p.free(1)
    assert p.n_free == 1 and p.alloc() == 1                       # the page that came back goes out again
    p.free(0)
    with pytest.raises(CacheError):
        p.free(0)                                                 # freed twice
    with pytest.raises(CacheError):
        p.free(7)
    assert p.peak_in_use == 3


def test_groups_follow_needs():
    m = _manager(window=6)
    assert len(m.groups) == 2 and m.groups[0].cache_ids == [0, 1] and m.groups[1].cache_ids == [2]
    assert m.group_of_cache[1] == (0, 1) and m.groups[1].window == 6


def test_one_page_per_page_size_positions_and_all_or_nothing():
    m = _manager(n_pages=5, page=4)
    m.admit("a")
    assert m.reserve("a", 9) and m.block_table("a", 0) == [0, 1, 2]
    m.advance("a", 9)
    assert m.reserve("a", 3) and len(m.block_table("a", 0)) == 3   # 12 positions still fit three pages
    m.advance("a", 3)
    m.admit("b")
    assert not m.reserve("b", 9)                                   # needs 3, only 2 free: nothing is taken
    assert m.pages_free() == [2] and m.block_table("b", 0) == []
    assert m.reserve("b", 8)
    assert not m.can_reserve([("a", 1)])
    m.release("a")
    assert m.pages_free() == [3]
    m.check_invariants()
    with pytest.raises(CacheError):
        m.release("a")
    with pytest.raises(CacheError):
        m.advance("b", 9)                                          # more than was reserved


def test_window_pages_go_back_and_table_keeps_holes():
    m = _manager(n_pages=8, page=4, window=6)
    m.admit("a")
    for n in (5, 1, 1, 6, 1, 1, 9):
        assert m.reserve("a", n)
        m.advance("a", n)
        L = m.length("a")
        t = m.block_table("a", 1)
        first_needed = max(0, L - 6 + 1) // 4
        assert all(p == -1 for p in t[:first_needed]) and all(p >= 0 for p in t[first_needed:])
        assert all(p >= 0 for p in m.block_table("a", 0))
        m.check_invariants()
    assert m.pages_in_use()[1] < m.pages_in_use()[0]
    m.release("a")
    assert m.pages_in_use() == [0, 0]


def test_unreserve_returns_only_the_unfilled_pages():
    m = _manager(n_pages=8, page=4)
    m.admit("a")
    m.reserve("a", 6); m.advance("a", 6)
    m.reserve("a", 9)
    assert len(m.block_table("a", 0)) == 4
    m.unreserve("a")
    assert len(m.block_table("a", 0)) == 2 and m.pages_free() == [6]
    m.check_invariants()


def test_state_slots_are_zeroed_and_reused():
    m = _manager(slots=2, with_state=True)
    m.make_storage(torch.float32, "cpu")
    a = m.admit("a")
    m.view(3)["s"][a.slot] += 5.0
    m.admit("b")
    with pytest.raises(CacheError):
        m.admit("c")                                               # no free slot
    m.release("a")
    c = m.admit("c")
    assert c.slot == a.slot and float(m.view(3)["s"][c.slot].abs().sum()) == 0.0
    m.check_invariants()
    v = m.view(0)
    assert v.k.shape == (16, 2, 4, 8) and v.group == 0 and m.view(1).k.data_ptr() != v.k.data_ptr()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = np.random.default_rng(seed)
    m = _manager(n_pages=12, page=4, slots=4, window=7)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.integers(0, 10)
        if op < 2 and len(live) < 4:
            m.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 8 and live:
            rid = list(live)[rng.integers(0, len(live))]
            n = int(rng.integers(1, 10))
            if m.can_reserve([(rid, n)]):
                assert m.reserve(rid, n)
                if rng.random() < 0.15:
                    m.unreserve(rid)
                else:
                    m.advance(rid, n); live[rid] += n
            else:
                before = m.pages_free()
                assert not m.reserve(rid, n) and m.pages_free() == before
        elif live:
            rid = list(live)[rng.integers(0, len(live))]
            m.release(rid); del live[rid]
        m.check_invariants()
        for rid, L in live.items():
            assert m.length(rid) == L
            full = m.block_table(rid, 0)
            assert len(full) >= -(-L // 4) and all(p >= 0 for p in full)
    for rid in list(live):
        m.release(rid)
    assert m.pages_in_use() == [0, 0]
    m.check_invariants()
