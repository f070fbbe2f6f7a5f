import random

import pytest

from sglang_c_b200.cache import CacheError, CacheManager, CacheNeed, PagePool, PagePoolError


def test_pool_is_lifo_and_all_or_nothing():
    p = PagePool(4)
    assert p.alloc(3) == [0, 1, 2]            # page 0 pops first, as in the reference's stack
    assert p.alloc(2) is None and p.n_free == 1
    p.unref(1)
    assert p.alloc(1) == [1]                  # a page given back is the next one handed out
    p.ref(0)
    p.unref(0)
    assert p.n_free == 1
    p.unref(0)
    assert p.n_free == 2
    with pytest.raises(PagePoolError):
        p.unref(0)                            # freed twice
    with pytest.raises(PagePoolError):
        p.ref(0)
    with pytest.raises(PagePoolError):
        p.unref(99)
    p.check()


def _mgr(n_pages=8, page_size=4, max_requests=3, window=None, n_calls=2):
    need = CacheNeed.paged_kv(2, 8, window)
    return CacheManager([need] * n_calls, [None] * n_calls, page_size, n_pages, max_requests)


def test_requests_grow_page_by_page_and_give_all_back():
    m = _mgr()
    assert m.add_request("a") == 0 and m.add_request("b") == 1
    assert m.extend("a", 5) and m.block_table(0, "a") == [0, 1]
    assert m.extend("b", 4) and m.block_table(0, "b") == [2]
    assert m.extend("a", 8) and m.block_table(0, "a") == [0, 1]      # still fits
    assert m.extend("a", 9) and m.block_table(0, "a") == [0, 1, 3]
    assert m.slot_of_position(0, "a", 8) == 3 * 4 + 0
    assert m.n_free_pages() == 4
    assert not m.extend("b", 4 + 4 * 5)                               # needs 5, 4 free: nothing changes
    assert m.block_table(0, "b") == [2] and m.length("b") == 4
    assert not m.can_extend_all([("a", 16), ("b", 17)])               # 1 + 4 pages > 4 free
    assert m.can_extend_all([("a", 16), ("b", 16)])                   # 1 + 3 pages fit exactly
    m.check()
    m.free_request("a")
    assert m.n_free_pages() == 7
    assert m.add_request("c") == 0                                     # slot reused
    assert m.extend("c", 1) and m.block_table(0, "c") == [3]           # LIFO: last freed first
    with pytest.raises(CacheError):
        m.free_request("a")                                            # freed twice
    with pytest.raises(CacheError):
        m.add_request("c")
    m.free_request("b")
    m.free_request("c")
    assert m.n_free_pages() == 8
    m.check()


def test_grow_by_one_and_its_undo():
    """The engine's ahead-of-time growth of a step of single tokens: one position more for every
    request, a page for those that begin one, and all of it taken back."""
    m = _mgr(n_pages=8)
    for r, n in (("a", 4), ("b", 6), ("c", 8)):
        m.add_request(r)
        assert m.extend(r, n)
    free, tables = m.n_free_pages(), {r: list(m.block_table(0, r)) for r in "abc"}
    reqs = ["a", "b", "c"]
    took = {0, 2}                                    # positions 4 and 8 begin pages
    assert m.can_extend_all([("a", 5), ("c", 9)])
    m.grow_by_one(reqs, took)
    assert [m.length(r) for r in reqs] == [5, 7, 9]
    assert m.n_free_pages() == free - 2 and len(m.block_table(0, "a")) == 2 and len(m.block_table(0, "c")) == 3
    m.check()
    m.shrink_by_one(reqs, took)
    assert [m.length(r) for r in reqs] == [4, 6, 8]
    assert m.n_free_pages() == free and {r: list(m.block_table(0, r)) for r in "abc"} == tables
    m.check()
    m.grow_by_one(reqs, took)                        # and kept this time
    for r in reqs:
        m.free_request(r)
    assert m.n_free_pages() == 8
    m.check()


def test_slots_run_out():
    m = _mgr(max_requests=2)
    assert m.add_request(1) is not None and m.add_request(2) is not None
    assert m.add_request(3) is None
    m.free_request(1)
    assert m.add_request(3) is not None
    m.check()


def test_window_pages_are_given_back_when_passed():
    m = _mgr(n_pages=4, page_size=4, window=6)
    m.add_request("w")
    assert m.extend("w", 10)                       # blocks 0,1,2
    assert m.block_table(0, "w") == [0, 1, 2]
    # next query is at position 10 and sees keys 5..10: block 0 (positions 0-3) has passed
    assert m.extend("w", 11)
    assert m.block_table(0, "w") == [-1, 1, 2]
    assert m.n_free_pages() == 2
    assert m.extend("w", 16)                       # block 3 takes the page block 0 gave back
    # old length 11: queries from position 11 see keys 6..: block 1 (4-7) still needed
    assert m.block_table(0, "w") == [-1, 1, 2, 0]
    assert m.extend("w", 17)                       # old length 16 -> first key 11 -> block 1 passes
    assert m.block_table(0, "w")[:3] == [-1, -1, 2]
    with pytest.raises(CacheError):
        m.slot_of_position(0, "w", 2)
    m.check()
    # a long sequence lives in a pool far smaller than its length
    for n in range(18, 200):
        assert m.extend("w", n), n
        m.check()
    m.free_request("w")
    assert m.n_free_pages() == 4


def test_groups_by_need_and_shared_caches():
    full = CacheNeed.paged_kv(2, 8)
    win = CacheNeed.paged_kv(2, 8, window=4)
    state = CacheNeed.state((3, 5))
    needs = [full, win, full, state, None, full]
    cache_of = [None, None, None, None, None, 0]
    m = CacheManager(needs, cache_of, 4, 6, 2)
    assert len(m.groups) == 3
    assert m.binding(0).group == m.binding(2).group == m.binding(5).group
    assert m.binding(1).group != m.binding(0).group
    assert m.binding(5).write is False and m.binding(0).write is True
    assert m.binding(4) is None and m.binding(3).kind == "state"
    m.add_request("x")
    assert m.extend("x", 9)
    assert m.block_table(m.binding(0).group, "x") == [0, 1, 2]
    assert len(m.block_table(m.binding(1).group, "x")) == 3
    with pytest.raises(CacheError):
        CacheManager([full, win], [None, 0], 4, 6, 2)          # shared cache with another need
    with pytest.raises(CacheError):
        CacheManager([None, full], [None, 0], 4, 6, 2)         # reads a call that keeps nothing


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    window = [None, 7, None, 5, 12, None][seed]
    m = _mgr(n_pages=12, page_size=4, max_requests=4, window=window)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            if m.add_request(next_id) is not None:
                live[next_id] = 0
            else:
                assert m.n_free_slots() == 0
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            n = live[r] + rng.choice([1, 1, 1, 2, 5, 9])
            free_before = m.n_free_pages()
            ok = m.extend(r, n)
            if ok:
                live[r] = n
            elif window is None:
                assert m.n_free_pages() == free_before      # a failed extend takes nothing
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        m.check()
        for r, n in live.items():
            assert m.length(r) == n
            table = m.block_table(0, r)
            assert len(table) >= (n + 3) // 4
            if window is None:
                assert all(p >= 0 for p in table)
    for r in list(live):
        m.free_request(r)
    assert m.n_free_pages() == 12 and m.n_free_slots() == 4
    m.check()
