"""The cache manager under random orders of requests (no GPU): no page is
lost, held twice or freed twice; window groups give pages back; growth is
all-or-nothing."""
import random

import pytest

from kipp_b200.cache import UNMAPPED, CacheManager, OutOfPages, OutOfSlots, PagePool, StateSlots
from kipp_b200.parts.base import PagedKVSpec

FULL = PagedKVSpec(2, 16)
WIN = PagedKVSpec(2, 16, window=10)


def test_pool_basics_and_reuse_order():
    p = PagePool(3)
    a, b, c = p.alloc("x"), p.alloc("x"), p.alloc("y")
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(OutOfPages):
        p.alloc("z")
    p.free(b, "x")
    with pytest.raises(RuntimeError, match="freed twice"):
        p.free(b, "x")
    with pytest.raises(RuntimeError, match="belongs to"):
        p.free(c, "x")
    p.free(a, "x")
    assert p.alloc("z") == b and p.alloc("z") == a          # freed pages come back in order
    p.check()


def test_slots():
    s = StateSlots(2)
    a, b = s.alloc("r1"), s.alloc("r2")
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfSlots):
        s.alloc("r3")
    s.free(a, "r1")
    with pytest.raises(RuntimeError):
        s.free(a, "r1")
    assert s.alloc("r3") == a
    s.check()


def test_groups_by_spec_and_block_tables():
    m = CacheManager({0: FULL, 1: WIN, 2: WIN, 3: FULL}, page_size=4, pages_per_group=8, max_requests=4)
    assert [g.cache_ids for g in m.groups] == [[0, 3], [1, 2]]
    assert m.group_of_cache == {0: (0, 0), 3: (0, 1), 1: (1, 0), 2: (1, 1)}
    m.admit("a")
    m.reserve([("a", 9)])
    m.advance("a", 9)
    assert m.table("a", 0) == [0, 1, 2] and m.table("a", 1) == [0, 1, 2]
    m.admit("b")
    m.reserve([("b", 3)])
    m.advance("b", 3)
    rows = m.block_table_rows(["b", "a"], 0)
    assert rows.tolist() == [[3, UNMAPPED, UNMAPPED], [0, 1, 2]] and rows.dtype.name == "int32"
    m.check()


def test_window_pages_are_given_back():
    m = CacheManager({0: FULL, 1: WIN}, page_size=4, pages_per_group={FULL: 16, WIN: 5}, max_requests=2)
    m.admit("a")
    length = 0
    for n in (7, 1, 1, 6, 2, 9, 1, 1, 1, 5, 8):
        m.reserve([("a", length + n)])
        # every position a token of this step may read is mapped in the window group
        lo = max(0, length - 10 + 1)
        for pos in range(lo, length + n):
            assert m.table("a", 1)[pos // 4] != UNMAPPED
        length += n
        m.advance("a", length)
        held = m.pages_held("a")
        assert held[0] == -(-length // 4)
        assert held[1] <= m.groups[1].peak_pages(10_000, 9)
        first_needed = max(0, length - 10 + 1)
        assert all(p == UNMAPPED for p in m.table("a", 1)[:first_needed // 4])
        m.check()
    assert length == 42 and m.pages_held("a")[1] <= 4      # 42 tokens passed through 5 pages
    m.release("a")
    assert m.free_pages() == [16, 5]


def test_all_or_nothing_growth():
    m = CacheManager({0: FULL}, page_size=4, pages_per_group=6, max_requests=3)
    for r in "abc":
        m.admit(r)
    m.reserve([("a", 8), ("b", 5)])
    m.advance("a", 8); m.advance("b", 5)
    before = (list(m.table("a", 0)), list(m.table("b", 0)), list(m.table("c", 0)), m.free_pages())
    with pytest.raises(OutOfPages):
        m.reserve([("c", 4), ("a", 12), ("b", 9)])          # needs 1 + 1 + 1 > 2 free
    assert (m.table("a", 0), m.table("b", 0), m.table("c", 0), m.free_pages()) == before
    m.check()
    m.reserve([("c", 4), ("a", 12)])                          # exactly the two free pages
    assert m.free_pages() == [0]
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = CacheManager({0: FULL, 1: WIN, 2: FULL}, page_size=rng.choice([2, 4, 8]),
                     pages_per_group={FULL: 24, WIN: 10}, max_requests=4)
    lengths: dict[str, int] = {}
    seen_pages = [set(), set()]
    reused = False
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(lengths) < 4:
            rid = f"r{next_id}"; next_id += 1
            m.admit(rid); lengths[rid] = 0
        elif action < 0.40 and lengths:
            rid = rng.choice(sorted(lengths))
            m.release(rid); del lengths[rid]
        elif action < 0.50 and lengths:
            # cut a request back: to nothing always works; to some length only while the
            # window group still holds what the next token would see
            rid = rng.choice(sorted(lengths))
            to = rng.choice([0, 0, rng.randint(0, lengths[rid])])
            held = [m.pages_held(rid), m.free_pages()]
            try:
                m.truncate(rid, to)
                lengths[rid] = to
            except ValueError:
                assert to > 0 and [m.pages_held(rid), m.free_pages()] == held
        elif lengths:
            batch = rng.sample(sorted(lengths), rng.randint(1, len(lengths)))
            wants = [(r, lengths[r] + rng.choice([1, 1, 1, 2, 5, 13])) for r in batch]
            snapshot = {r: [list(m.table(r, g)) for g in range(2)] for r in lengths}
            free_before = m.free_pages()
            try:
                m.reserve(wants)
            except OutOfPages:
                assert m.free_pages() == free_before
                for r in lengths:
                    assert [list(m.table(r, g)) for g in range(2)] == snapshot[r]
                victim = max(lengths, key=lengths.get)
                m.release(victim); del lengths[victim]
            else:
                for r, n in wants:
                    for g in range(2):
                        for p in m.table(r, g):
                            if p != UNMAPPED:
                                if p in seen_pages[g] and p not in snapshot[r][g]:
                                    reused = True
                                seen_pages[g].add(p)
                    m.advance(r, n); lengths[r] = n
        m.check()
        for r, n in lengths.items():
            assert m.length(r) == n
            assert m.pages_held(r)[0] == -(-n // m.page_size)
    for r in list(lengths):
        m.release(r)
    m.check()
    assert m.free_pages() == [24, 10] and m.slots.free_slots == 4
    assert reused                                               # pages were used again


def test_truncate_gives_back_the_pages_past_the_new_length():
    m = CacheManager({0: FULL, 1: FULL}, page_size=4, pages_per_group={FULL: 8}, max_requests=2)
    m.admit("a")
    m.reserve([("a", 21)]); m.advance("a", 21)
    assert m.pages_held("a")[0] == 6
    m.truncate("a", 9)                                      # pages 0..2 stay
    assert m.length("a") == 9 and m.pages_held("a")[0] == 3 and m.free_pages()[0] == 5
    m.check()
    m.reserve([("a", 10)]); m.advance("a", 10)              # goes on from there
    with pytest.raises(ValueError):
        m.truncate("a", 11)
    m.truncate("a", 0)
    assert m.pages_held("a") == [0] and m.free_pages() == [8]
    m.reserve([("a", 3)]); m.advance("a", 3)
    m.check()
    # a window that has given pages back cannot be cut back into them
    w = CacheManager({0: FULL, 1: WIN}, page_size=4, pages_per_group={FULL: 8, WIN: 8}, max_requests=2)
    w.admit("b")
    w.reserve([("b", 30)]); w.advance("b", 30)
    assert w.pages_held("b")[1] < 8                         # the window let go of early pages
    held, free = w.pages_held("b"), w.free_pages()
    with pytest.raises(ValueError, match="window"):
        w.truncate("b", 5)
    assert w.length("b") == 30 and w.pages_held("b") == held and w.free_pages() == free
    w.truncate("b", 29)                                     # its window still lies in held pages
    w.check()
    w.truncate("b", 0)
    assert w.free_pages() == [8, 8]
    w.reserve([("b", 6)]); w.advance("b", 6)
    w.check()


def test_errors_leave_everything_as_it_was():
    """Whatever refuses a reserve (a pool that is empty, a request that would shrink),
    the pages the call had taken are back and the tables are as before; rows narrower
    than a table are refused; unknown requests are KeyErrors."""
    m = CacheManager({0: FULL}, page_size=4, pages_per_group=8, max_requests=2)
    m.admit("a"); m.admit("b")
    with pytest.raises(OutOfSlots):
        m.admit("c")
    assert "c" not in m and m.live_requests() == ["a", "b"]
    m.reserve([("a", 9)]); m.advance("a", 9)
    before = (m.table("a", 0), m.table("b", 0), m.free_pages())
    with pytest.raises(ValueError):
        m.reserve([("b", 7), ("a", 3)])                      # b would get pages, then a shrinks
    assert (m.table("a", 0), m.table("b", 0), m.free_pages()) == before
    with pytest.raises(ValueError):
        m.block_table_rows(["a"], 0, width=2)                # a holds three pages
    assert m.block_table_rows(["a", "b"], 0, width=4).tolist() == [[0, 1, 2, UNMAPPED], [UNMAPPED] * 4]
    for call in (lambda: m.length("zz"), lambda: m.reserve([("zz", 1)]), lambda: m.release("zz")):
        with pytest.raises(KeyError):
            call()
    assert m.groups[0].pool.owner(1) == "a" and m.groups[0].pool.owner(5) is None
    m.release("a"); m.release("b")
    m.check()
    assert m.free_pages() == [8] and m.slots.free_slots == 2
