"""The cache manager on the CPU: pages, block tables, windows, slots, under random request orders."""
import random

import pytest

from gesso_b200.cache import FREED, CacheManager, IndexPool, PagedGroupSpec
from gesso_b200.errors import ErrorCode, GessoError


def make(num_pages=8, page_size=4, slots=3, ctx=64, window=None):
    groups = [PagedGroupSpec("full", None)]
    if window:
        groups.append(PagedGroupSpec("win", window))
    return CacheManager(groups, page_size, num_pages, slots, ctx)


def test_pool_hands_out_and_takes_back():
    p = IndexPool(3, "page")
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert sorted([a, b, c]) == [0, 1, 2] and p.free_count == 0
    with pytest.raises(GessoError) as e:
        p.alloc()
    assert e.value.code == ErrorCode.RESOURCE_LIMIT
    p.free(b)
    assert p.alloc() == b                      # last freed, first reused
    with pytest.raises(GessoError):
        p.free(7)
    p.free(a)
    with pytest.raises(GessoError):
        p.free(a)                              # freed twice


def test_append_across_page_borders():
    m = make()
    m.admit("r")
    for n_new, pages in ((3, 1), (1, 1), (1, 2), (7, 3), (4, 4)):
        m.reserve("r", n_new)
        m.commit("r", n_new)
        assert len(m.block_table("r", 0)) == pages
        m.check_invariants()
    assert m.length("r") == 16 and m.pages_in_use() == [4]
    m.release("r")
    assert m.pages_in_use() == [0] and m.slots_in_use() == 0
    m.check_invariants()


def test_exhaustion_is_a_typed_error_and_changes_nothing():
    m = make(num_pages=2)
    m.admit("a")
    m.reserve("a", 8)
    m.commit("a", 8)
    m.admit("b")
    assert not m.can_reserve("b", 1)
    with pytest.raises(GessoError) as e:
        m.reserve("b", 1)
    assert e.value.code == ErrorCode.RESOURCE_LIMIT
    assert m.block_table("b", 0) == [] and m.pages_in_use() == [2]
    m.check_invariants()


def test_context_length_limit():
    m = make(ctx=8)
    m.admit("x")
    with pytest.raises(GessoError) as e:
        m.reserve("x", 9)
    assert e.value.code == ErrorCode.RESOURCE_LIMIT and "context" in str(e.value)


def test_slots_and_fresh_flag():
    m = make(slots=2)
    s0 = m.admit("a")
    s1 = m.admit("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(GessoError):
        m.admit("c")
    with pytest.raises(GessoError):
        m.admit("a")                           # already live
    assert m.take_fresh("a") is True and m.take_fresh("a") is False
    m.release("a")
    assert m.admit("c") == s0 and m.take_fresh("c") is True     # a reused slot is fresh again
    with pytest.raises(GessoError):
        m.length("a")


def test_window_group_gives_pages_back():
    m = make(num_pages=8, page_size=4, window=6)
    m.admit("r")
    m.reserve("r", 20)
    assert len(m.block_table("r", 1)) == 5
    m.commit("r", 20)
    # the next query sits at position 20 and reads keys >= 15: pages 0..2 (positions 0..11) are dead
    assert m.block_table("r", 1)[:3] == [FREED] * 3 and FREED not in m.block_table("r", 1)[3:]
    assert FREED not in m.block_table("r", 0)
    assert m.pages_in_use() == [5, 2]
    for _ in range(8):
        m.reserve("r", 1)
        m.commit("r", 1)
        m.check_invariants()
    assert m.pages_in_use()[1] <= 3
    m.release("r")
    assert m.pages_in_use() == [0, 0]
    m.check_invariants()


def test_all_groups_or_none():
    m = CacheManager([PagedGroupSpec("a"), PagedGroupSpec("b")], 4, [4, 1], 2, 64)
    m.admit("r")
    with pytest.raises(GessoError):
        m.reserve("r", 8)                      # group b has one page only
    assert m.pages_in_use() == [0, 0]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = make(num_pages=12, page_size=4, slots=4, ctx=40, window=9 if seed % 2 else None)
    live, next_id, reused = {}, 0, set()
    seen_pages = set()
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 5, 9])
            if m.can_reserve(r, n):
                m.reserve(r, n)
                for p in m.block_table(r, 0):
                    if p in seen_pages:
                        reused.add(p)
                m.commit(r, n)
                live[r] += n
                assert m.length(r) == live[r]
            else:
                with pytest.raises(GessoError):
                    m.reserve(r, n)
        elif live:
            r = rng.choice(list(live))
            seen_pages.update(p for p in m.block_table(r, 0) if p != FREED)
            m.release(r)
            del live[r]
        m.check_invariants()
        held = sum(len([p for p in m.block_table(r, 0) if p != FREED]) for r in live)
        assert held == m.pages_in_use()[0]
        for r in live:   # full group: exactly the pages the length needs (or reserved ahead)
            assert len(m.block_table(r, 0)) >= (live[r] + 3) // 4
    for r in list(live):
        m.release(r)
    assert m.pages_in_use() == [0] * len(m.groups) and m.slots_in_use() == 0
    assert reused, "pages were never used again: the pool is too large for this test"


def test_single_token_reservation_equals_the_general_one():
    """The decoding fast path hands out the same pages as ``reserve`` one request at a time, is all or
    nothing, and reports a fresh slot exactly once."""
    a, b = make(num_pages=14, page_size=4, slots=3, ctx=40, window=6), make(num_pages=14, page_size=4, slots=3, ctx=40, window=6)
    for m in (a, b):
        for r in ("x", "y", "z"):
            m.admit(r)
    fresh_seen = []
    for step in range(13):
        starts, slots, fresh, rows = a.reserve_single_tokens(["x", "y", "z"])
        fresh_seen += fresh
        for r in ("x", "y", "z"):
            b.reserve(r, 1)
        assert starts == [b.length(r) for r in ("x", "y", "z")] and slots == [b.slot(r) for r in ("x", "y", "z")]
        for g in range(2):
            for i, r in enumerate(("x", "y", "z")):
                assert rows[g][i].tolist()[:len(b.block_table(r, g))] == b.block_table(r, g)
                assert a.block_table(r, g) == b.block_table(r, g)
        for r in ("x", "y", "z"):
            a.commit(r, 1)
            b.commit(r, 1)
        a.check_invariants()
    assert sorted(fresh_seen) == [0, 1, 2]
    # all or nothing: 2 pages, three requests at a page border need 3 pages
    c = make(num_pages=2, page_size=4, slots=3, ctx=40)
    for r in ("x", "y", "z"):
        c.admit(r)
    with pytest.raises(GessoError):
        c.reserve_single_tokens(["x", "y", "z"])
    assert c.pages_in_use() == [0]
    with pytest.raises(GessoError):
        c.reserve_single_tokens(["nobody"])


def test_step_reservation_equals_the_general_one():
    """``reserve_step`` (a whole mixed step in one native call) hands out the same pages as ``reserve``
    request by request, is all or nothing, refuses a request named twice and reports fresh slots once."""
    a, b = make(num_pages=20, page_size=4, slots=3, ctx=40, window=6), make(num_pages=20, page_size=4, slots=3, ctx=40, window=6)
    for m in (a, b):
        for r in ("x", "y", "z"):
            m.admit(r)
    fresh_seen = []
    for news in ([5, 1, 9], [1, 1, 1], [3, 7, 1], [8, 2, 4]):
        starts, slots, fresh, max_kv, rows = a.reserve_step(["x", "y", "z"], news)
        fresh_seen += fresh
        for r, k in zip(("x", "y", "z"), news):
            b.reserve(r, k)
        assert starts == [b.length(r) for r in ("x", "y", "z")] and slots == [b.slot(r) for r in ("x", "y", "z")]
        assert max_kv == max(b.length(r) + k for r, k in zip(("x", "y", "z"), news))
        for g in range(2):
            for i, r in enumerate(("x", "y", "z")):
                assert a.block_table(r, g) == b.block_table(r, g)
                assert rows[g][i].tolist()[:len(b.block_table(r, g))] == b.block_table(r, g)
        a.commit_step(["x", "y", "z"], news)
        for r, k in zip(("x", "y", "z"), news):
            b.commit(r, k)
        assert [a.length(r) for r in ("x", "y", "z")] == [b.length(r) for r in ("x", "y", "z")]
        a.check_invariants()
    assert sorted(fresh_seen) == [0, 1, 2]
    c = make(num_pages=3, page_size=4, slots=3, ctx=40)
    for r in ("x", "y"):
        c.admit(r)
    with pytest.raises(GessoError):
        c.reserve_step(["x", "y"], [9, 5])          # 3 + 2 pages wanted, 3 there: nobody gets any
    assert c.pages_in_use() == [0]
    with pytest.raises(GessoError):
        c.reserve_step(["x", "x"], [1, 1])
    with pytest.raises(GessoError):
        c.reserve_step(["x", "y"], [41, 1])         # beyond the context length
    assert c.pages_in_use() == [0]
    c.reserve_step(["x", "y"], [8, 4])
    assert c.pages_in_use() == [3]
