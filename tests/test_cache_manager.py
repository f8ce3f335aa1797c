"""Cache manager: no page lost, held twice or freed twice; windows give pages back; slots."""

import random

import pytest

from qwen3_from_scratch_b200.cache import CacheError, CacheManager, OutOfPages, OutOfSlots, layout_of
from qwen3_from_scratch_b200.parts.base import KVCacheSpec, StateSpec

FULL = KVCacheSpec(2, 16, None)
WIN = KVCacheSpec(2, 16, 10)


def manager(specs, page_size=4, num_pages=8, max_seqs=3):
    return CacheManager(layout_of(dict(enumerate(specs))), page_size, num_pages, max_seqs)


def test_layers_with_equal_needs_share_a_group():
    layout = layout_of({0: FULL, 1: WIN, 2: FULL, 3: StateSpec((4,)), 4: None, 5: WIN})
    assert [g.cache_ids for g in layout.groups] == [[0, 2], [1, 5]]
    assert list(layout.states) == [3]
    assert layout.group_of(5) == 1


def test_pages_grow_with_the_request_and_come_back():
    m = manager([FULL, FULL])
    m.open("a")
    m.reserve("a", 5)
    assert m.table(0, "a") == [0, 1] and m.free_pages() == 6
    m.advance("a", 5)
    m.reserve("a", 8)  # still two pages
    assert m.free_pages() == 6
    m.reserve("a", 9)
    assert m.table(0, "a") == [0, 1, 2]
    m.advance("a", 9)
    m.check()
    m.close("a")
    assert m.free_pages() == 8 and m.free_slots() == 3
    m.open("b")
    m.reserve("b", 1)
    assert m.table(0, "b") == [2]  # the page given back last is handed out first
    m.check()


def test_reserve_takes_nothing_when_it_cannot_take_all():
    m = manager([FULL, WIN], num_pages=3)
    m.open("a")
    m.reserve("a", 8)
    m.open("b")
    assert not m.can_reserve("b", 8)
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert m.free_pages(0) == 1 and m.free_pages(1) == 1 and m.table(0, "b") == []
    m.check()


def test_window_gives_pages_back_as_it_passes():
    m = manager([WIN], page_size=4, num_pages=6)  # window of 10 tokens
    m.open("a")
    held = []
    for length in range(1, 41):
        m.reserve("a", length)
        m.advance("a", length)
        m.check()
        table = m.table(0, "a")
        live = [p for p in table if p >= 0]
        held.append(len(live))
        # the next query (position `length`) reads keys > length - 10: their pages must be live
        first_key = max(0, length - 10 + 1)
        for pos in range(first_key, length):
            assert table[pos // 4] >= 0
        # and nothing older than the page of the first key is kept
        assert all(p < 0 for p in table[: first_key // 4])
    assert max(held) <= 4  # (window + page) / page, never the whole sequence
    assert len(m.table(0, "a")) == 10


def test_window_portion_keeps_what_its_first_query_reads():
    m = manager([WIN], page_size=4, num_pages=16)
    m.open("a")
    m.reserve("a", 30)
    m.advance("a", 30)  # next query at 30 reads keys 21..29 -> pages 5.. ; pages 0..4 given back
    assert [p >= 0 for p in m.table(0, "a")] == [False] * 5 + [True] * 3
    m.reserve("a", 37)
    assert len(m.table(0, "a")) == 10


def test_freeing_twice_and_foreign_frees_are_errors():
    m = manager([FULL])
    m.open("a")
    m.reserve("a", 4)
    m.close("a")
    with pytest.raises(CacheError, match="not open"):
        m.close("a")
    with pytest.raises(CacheError, match="already open"):
        m.open("b") or m.open("b")
    pool = m._pools[0]
    with pytest.raises(CacheError, match="freed twice"):
        pool.give_back(0, "a")
    page = pool.take("x")
    with pytest.raises(CacheError, match="held by"):
        pool.give_back(page, "y")


def test_slots():
    m = manager([FULL, StateSpec((8,))], max_seqs=2)
    assert m.open("a") == 0 and m.open("b") == 1
    with pytest.raises(OutOfSlots):
        m.open("c")
    m.close("a")
    assert m.open("c") == 0
    m.check()


def test_advance_beyond_reserved_pages_is_refused():
    m = manager([FULL])
    m.open("a")
    m.reserve("a", 4)
    with pytest.raises(CacheError, match="beyond"):
        m.advance("a", 5)
    with pytest.raises(CacheError, match="shrink"):
        m.advance("a", 4) or m.advance("a", 3)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    specs = [FULL, WIN, FULL, KVCacheSpec(1, 32, 7), StateSpec((3,))]
    page, pages = rng.choice([2, 4, 16]), rng.choice([12, 40])
    m = CacheManager(layout_of(dict(enumerate(specs))), page, pages, max_seqs=5)
    m.freed_log = []
    lengths = {}
    next_id = 0
    given_back = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and m.free_slots():
            m.open(next_id)
            lengths[next_id] = 0
            next_id += 1
        elif action < 0.85 and lengths:
            req = rng.choice(list(lengths))
            new = lengths[req] + rng.choice([1, 1, 1, 2, 5, 13])
            if m.can_reserve(req, new):
                m.reserve(req, new)
                m.advance(req, new)
                lengths[req] = new
            else:
                free_before = [m.free_pages(g) for g in range(3)]
                with pytest.raises(OutOfPages):
                    m.reserve(req, new)
                assert free_before == [m.free_pages(g) for g in range(3)]
        elif lengths:
            req = rng.choice(list(lengths))
            m.close(req)
            del lengths[req]
        m.check()
        for req, n in lengths.items():
            assert m.length(req) == n
            full = m.table(0, req)
            assert len(full) == -(-n // page) and all(p >= 0 for p in full)
    for req in list(lengths):
        m.close(req)
    m.check()
    assert all(m.free_pages(g) == pages for g in range(3)) and m.free_slots() == 5
    assert len(m.freed_log) > 0
