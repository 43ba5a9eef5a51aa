"""The cache manager's books: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; slots."""

import random

import numpy as np
import pytest

from tokasaurus_b200.cache import CacheManager, NoSlotError, NoSpaceError, PageAllocator, StateSlotAllocator
from tokasaurus_b200.parts.base import PagedCacheNeed, StateNeed

FULL = PagedCacheNeed(2, 16)
WIN = PagedCacheNeed(2, 16, window=20)


def test_allocator_basics():
    a = PageAllocator(4)
    p = a.allocate(3, "x")
    assert sorted(p) == [0, 1, 2] and a.num_free == 1
    with pytest.raises(NoSpaceError):
        a.allocate(2, "y")
    assert a.num_free == 1  # a refused request changes nothing
    a.release(p[:1], "x")
    with pytest.raises(ValueError, match="twice"):
        a.release(p[:1], "x")
    with pytest.raises(ValueError, match="belongs"):
        a.release(p[1:2], "y")
    assert a.allocate(1, "z") == p[:1]  # the page given back is handed out next
    a.check()


def test_slots():
    s = StateSlotAllocator(2)
    a, b = s.allocate("a"), s.allocate("b")
    assert {a, b} == {0, 1}
    with pytest.raises(NoSlotError):
        s.allocate("c")
    s.release(a, "a")
    with pytest.raises(ValueError):
        s.release(a, "a")
    assert s.allocate("c") == a
    s.check()


def test_groups_follow_needs():
    m = CacheManager({0: FULL, 1: WIN, 2: FULL, 3: StateNeed((4,)), 4: None, 5: WIN}, page_size=8, num_pages=10,
                     max_requests=3)
    assert [g.entries for g in m.groups] == [[0, 2], [1, 5]]
    assert m.group_of(2) == 0 and m.group_of(5) == 1 and m.group_of(3) is None
    assert m.layer_cache(4) is None and m.layer_cache(3).state is None


def test_capacity_is_all_or_nothing():
    m = CacheManager({0: FULL, 1: WIN}, page_size=4, num_pages=5, max_requests=4)
    m.admit("a")
    m.ensure_capacity("a", 12)
    m.admit("b")
    with pytest.raises(NoSpaceError):
        m.ensure_capacity("b", 12)
    assert m.table("b", 0) == [] and m.table("b", 1) == [] and m.num_free_pages() == [2, 2]
    m.ensure_capacity("b", 8)
    m.check()
    m.free("a")
    m.ensure_capacity("b", 20)
    assert m.num_free_pages() == [0, 0]
    m.free("b")
    assert m.num_free_pages() == [5, 5]
    m.check()


def test_window_gives_pages_back_and_they_are_reused():
    m = CacheManager({0: FULL, 1: WIN}, page_size=8, num_pages=16, max_requests=2)
    m.admit("a")
    m.ensure_capacity("a", 64)
    assert m.num_free_pages() == [8, 8]
    # after 64 tokens the next query (position >= 64) sees keys > 64 - 20 = 44, i.e. from 45 on: pages 0..4 are dead
    assert m.release_behind_window("a", 64) == 5
    assert m.table("a", 1)[:5] == [-1] * 5 and m.num_free_pages() == [8, 13]
    assert m.release_behind_window("a", 64) == 0
    m.check()
    m.admit("b")
    m.ensure_capacity("b", 64)
    given_back = set(range(16)) - set(p for p in m.table("a", 1) if p >= 0) - set(range(8, 16))
    assert len(given_back) == 5 and given_back <= set(m.table("b", 1))  # pages that came back are handed out first
    m.free("a")
    m.free("b")
    assert m.num_free_pages() == [16, 16]
    m.check()


def test_windowed_groups_fill_portion_by_portion_in_a_pool_of_their_own():
    """With the step's token limit known, a windowed group's pool holds what the request slots can hold at once
    (window 20 + 16 tokens a step + 1 ahead = 37 tokens -> 5 pages, + 1: 6 a request), and a prompt that is
    longer than that pool passes through it while the full group holds all of it from the start."""
    m = CacheManager({0: FULL, 1: WIN}, page_size=8, num_pages=64, max_requests=2, max_step_tokens=16)
    assert [g.allocator.num_pages for g in m.groups] == [64, 12]
    m.admit("a")
    with pytest.raises(NoSpaceError):
        m.ensure_capacity("a", 200)  # all of it at once does not fit the windowed pool, and nothing is taken
    assert m.num_free_pages() == [64, 12]
    done = 0
    while done < 200:
        n = min(16, 200 - done)
        assert m.can_hold("a", 200, windowed_tokens=done + n)
        m.ensure_capacity("a", 200, windowed_tokens=done + n)
        assert len(m.table("a", 0)) == 25 and len(m.table("a", 1)) == -(-(done + n) // 8)
        done += n
        m.release_behind_window("a", done)
        assert sum(p >= 0 for p in m.table("a", 1)) <= 6
        m.check()
    m.free("a")
    assert m.num_free_pages() == [64, 12]


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = CacheManager({0: FULL, 1: WIN, 2: FULL}, page_size=4, num_pages=40, max_requests=6)
    live: dict[str, int] = {}
    n = 0
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and len(live) < 6:
            rid = f"q{n}"
            n += 1
            m.admit(rid)
            live[rid] = 0
        elif r < 0.8 and live:
            rid = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 7, 23])
            try:
                m.ensure_capacity(rid, live[rid] + grow)
                live[rid] += grow
                m.release_behind_window(rid, live[rid])
            except NoSpaceError:
                victim = rng.choice(list(live))
                m.free(victim)
                del live[victim]
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        for rid, length in live.items():
            assert len(m.table(rid, 0)) == -(-length // 4)
            assert all(p >= 0 for p in m.table(rid, 0))
            win = m.table(rid, 1)
            first_visible = max(0, length - 20 + 1)
            assert all(p >= 0 for p in win[first_visible // 4:])  # what can still be seen has a page
    for rid in list(live):
        m.free(rid)
    assert m.num_free_pages() == [40, 40]
    assert m.slots.num_free == 6
    with pytest.raises(KeyError):
        m.free("q0")


def test_decode_steps_are_laid_out_whole_and_equal_the_general_layout():
    """A step of single tokens from the device is laid out by array operations; every array equals what the
    request-by-request layout makes of the same entries (two cache groups, one windowed with pages given back)."""
    from dataclasses import fields
    from tokasaurus_b200.engine.batch import StepEntry, _decode_host_batch, _general_host_batch, build_host_batch

    m = CacheManager({0: FULL, 1: WIN}, page_size=8, num_pages=64, max_requests=8)
    rng = random.Random(3)
    entries = []
    for i in range(7):
        rid, n = f"r{i}", rng.randint(0, 70)
        m.admit(rid)
        m.ensure_capacity(rid, n + 1)
        m.release_behind_window(rid, n)
        entries.append(StepEntry(rid, None, n, [0]))
    fast, slow = _decode_host_batch(entries, m), _general_host_batch(entries, m)
    for f in fields(fast):
        a, b = getattr(fast, f.name), getattr(slow, f.name)
        if isinstance(a, list) and a and isinstance(a[0], np.ndarray):
            assert all(np.array_equal(x, y) and x.dtype == y.dtype for x, y in zip(a, b)), f.name
        elif isinstance(a, np.ndarray):
            assert np.array_equal(a, b) and a.dtype == b.dtype, f.name
        else:
            assert a == b, f.name
    assert build_host_batch(entries, m).token_ids.tolist() == [-1] * 7
    with pytest.raises(ValueError, match="twice"):
        build_host_batch(entries + [entries[0]], m)
    m.free("r0")
    m.admit("short")
    with pytest.raises(ValueError, match="holds 0 pages"):
        build_host_batch([StepEntry("short", None, 3, [0])], m)
