"""The cache manager without a device: no page is lost, held twice or freed twice under random
orders of requests; windows give pages back; groups have pools of their own."""
import random

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from mlx_lm_b200.cache import CacheManager, NoFreeSlot, OutOfPages, PagePool
from mlx_lm_b200.parts import PagedKVSpec, StateSpec

FULL = PagedKVSpec(4, 16, None)
WIN = PagedKVSpec(2, 32, 40)


def test_pool_refuses_double_free_and_exhaustion():
    p = PagePool(3)
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert sorted([a, b, c]) == [0, 1, 2] and p.n_free == 0
    with pytest.raises(OutOfPages):
        p.alloc()
    p.free(b)
    with pytest.raises(RuntimeError):
        p.free(b)
    assert p.alloc() == b          # the page freed last is taken first
    with pytest.raises(ValueError):
        p.free(7)


def test_groups_by_need():
    m = CacheManager({0: FULL, 1: WIN, 2: FULL, 3: StateSpec((8,)), 4: WIN}, page_size=16, n_pages=10, max_requests=2,
                     max_len=256)
    assert [g.cache_ids for g in m.kv_groups] == [[0, 2], [1, 4]]
    assert [g.cache_ids for g in m.state_groups] == [[3]]
    assert m.where(2) == ("kv", 0) and m.where(4) == ("kv", 1) and m.where(3) == ("state", 0)


def test_reserve_commit_truncate_release():
    m = CacheManager({0: FULL}, page_size=16, n_pages=6, max_requests=2, max_len=128)
    m.add_request("a")
    assert m.pages_needed("a", 17) == [2]
    assert m.reserve("a", 17) == 0
    m.commit("a")
    assert m.length("a") == 17 and m.pages_in_use() == [2]
    assert m.reserve("a", 15) == 17        # fills page 2 exactly: no new page
    m.commit("a")
    assert m.pages_in_use() == [2]
    assert m.reserve("a", 1) == 32
    m.commit("a")
    assert m.pages_in_use() == [3]
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 16 * 3 + 1)         # needs 4, 3 are free: nothing is taken
    assert m.pages_in_use() == [3]
    assert m.can_reserve([("b", 48)]) and not m.can_reserve([("b", 48), ("a", 16)])
    m.truncate("a", 16)
    assert m.length("a") == 16 and m.pages_in_use() == [1]
    with pytest.raises(NoFreeSlot):
        m.add_request("c")
    bt = m.block_table(0, ["a", "b"])
    assert bt.shape == (2, 8) and bt[0, 0] >= 0 and (bt[0, 1:] == -1).all() and (bt[1] == -1).all()
    m.release("a")
    m.release("b")
    assert m.pages_in_use() == [0]
    m.check()
    m.add_request("d")
    with pytest.raises(ValueError):
        m.reserve("d", 129)              # beyond the maximum length


def test_window_gives_pages_back():
    m = CacheManager({0: WIN}, page_size=16, n_pages=8, max_requests=1, max_len=1024)
    m.add_request("a")
    m.reserve("a", 100)
    assert m.pages_in_use() == [7]           # the whole portion needs its pages during the step
    m.commit("a")
    # next query is position 100; it needs keys 61..100, so pages 0..2 (keys 0..47) go back
    assert m.pages_in_use() == [4]
    assert list(m.block_table(0, ["a"])[0, :7]) [:3] == [-1, -1, -1]
    for _ in range(300):
        m.reserve("a", 1)
        m.commit("a")
        assert m.pages_in_use()[0] <= 4
        m.check()
    m.release("a")
    assert m.pages_in_use() == [0]


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 10 ** 6), st.sampled_from([8, 16, 64]), st.integers(4, 40))
def test_random_orders_never_lose_or_double_book(seed, page, n_pages):
    rng = random.Random(seed)
    m = CacheManager({0: FULL, 1: WIN, 2: StateSpec((4,))}, page_size=page, n_pages=n_pages, max_requests=4,
                     max_len=page * n_pages)
    live = {}
    for it in range(200):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{it}"
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, page, page + 3, 3 * page])
            if live[rid] + n > m.max_len:
                continue
            try:
                start = m.reserve(rid, n)
            except OutOfPages:
                before = m.pages_in_use()
                m.check()
                assert m.pages_in_use() == before
                continue
            assert start == live[rid]
            m.commit(rid)
            live[rid] += n
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            full = m.requests[rid].pages[0]
            assert len(full) == (n + page - 1) // page and all(p >= 0 for p in full)
            win = m.requests[rid].pages[1]
            first_needed = max(0, n - 40 + 1) // page
            assert all(p >= 0 for p in win[first_needed:]) and all(p < 0 for p in win[:first_needed])
    for rid in list(live):
        m.release(rid)
    m.check()
    assert m.pages_in_use() == [0, 0] and m.pages_free() == [n_pages, n_pages]


def test_rollback_undoes_a_reservation():
    """A step that failed gives its pages back and leaves the lengths where they were."""
    m = CacheManager({0: FULL, 1: WIN}, page_size=16, n_pages=8, max_requests=3, max_len=256)
    m.add_request("a")
    m.add_request("b")
    m.reserve("a", 20)
    m.commit("a")
    before = (m.pages_in_use(), m.length("a"), m.length("b"), list(m.requests["a"].pages[0]))
    m.reserve("a", 30)                     # crosses two page edges
    m.reserve("b", 5)
    assert m.pages_in_use() != before[0]
    m.rollback("a")
    m.rollback("b")
    m.check()
    assert (m.pages_in_use(), m.length("a"), m.length("b"), list(m.requests["a"].pages[0])) == before
    assert m.requests["a"].reserved == 0 and m.requests["b"].pages == [[], []]
    m.rollback("b")                        # nothing reserved: nothing happens
    assert m.reserve("a", 30) == 20        # and the request goes on from where it was
    m.commit("a")
    m.check()
    assert m.length("a") == 50
