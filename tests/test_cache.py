"""The cache manager on the host: no page lost, held twice or freed twice, under
random orders of requests; reuse order; windows; state slots."""

import random

import pytest

from redline_b200.cache import CacheError, CacheManager, GroupInfo, PageAllocator
from redline_b200.parts.spec import CacheSpec


def manager(pages=(9,), window=(0,), page_size=16, slots=4):
    groups = [GroupInfo(CacheSpec.keys_values("window" if w else "full", 2, 64, w), [i]) for i, w in enumerate(window)]
    return CacheManager(groups, list(pages), page_size, slots)


def test_allocator_order_exhaustion_and_double_free():
    a = PageAllocator(5)
    assert a.num_usable == 4 and [a.allocate() for _ in range(4)] == [1, 2, 3, 4]   # page 0 is reserved
    assert a.allocate() == -1
    a.free([3, 1])
    assert [a.allocate(), a.allocate()] == [3, 1]      # first of the freed list comes back first
    with pytest.raises(CacheError, match="twice"):
        a.free([2, 2])
    with pytest.raises(CacheError, match="not a page"):
        a.free([0])
    with pytest.raises(CacheError):
        PageAllocator(1)


def test_reserve_is_all_or_nothing_and_close_returns_everything():
    m = manager(pages=(6, 4), window=(0, 0))
    a = m.open("a")
    assert m.reserve(a, 40) and a.tables == [[1, 2, 3], [1, 2, 3]]
    b = m.open("b")
    assert not m.reserve(b, 17)            # group 1 has no page left: group 0's are given back
    assert b.tables == [[], []] and m.num_free_pages(0) == 2 and m.num_free_pages(1) == 0
    m.check_invariants()
    assert m.slot(a, 0, 37) == 3 * 16 + 5
    m.close("a")
    assert m.reserve(b, 33) and b.tables[0] == [1, 2, 3]   # LIFO: the same pages, in table order
    m.close("b")
    assert m.num_free_pages(0) == 5 and m.num_free_pages(1) == 3
    with pytest.raises(CacheError):
        m.close("b")
    with pytest.raises(CacheError):
        m.get("a")


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager(pages=(20, 20), window=(0, 40))
    r = m.open("r")
    assert m.reserve(r, 100)
    assert m.release_passed(r, 39) == 0
    # after 56 tokens the next position is 56 and sees keys 17..56: page 0 (keys 0..15) is dead
    assert m.release_passed(r, 56) == 1 and r.tables[1][0] == 0 and r.released_upto == [0, 1]
    assert m.release_passed(r, 100) == 2 and r.tables[1][:3] == [0, 0, 0] and r.tables[0][0] != 0
    m.check_invariants()
    assert m.reserve(r, 130) and len(r.tables[1]) == 9
    m.close("r")
    assert m.num_free_pages(0) == 19 and m.num_free_pages(1) == 19
    m.check_invariants()


def test_state_slots():
    m = manager(slots=2)
    seen = []
    m.on_open = lambda rc: seen.append(rc.state_slot)
    a, b = m.open("a"), m.open("b")
    assert {a.state_slot, b.state_slot} == {0, 1} and seen == [a.state_slot, b.state_slot]
    with pytest.raises(CacheError, match="state slot"):
        m.open("c")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    m.close("a")
    assert m.open("c").state_slot == a.state_slot
    m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = manager(pages=(14, 11), window=(0, 24), slots=5)
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            k = f"r{step}"
            live[k] = 0
            m.open(k)
        elif op < 0.75 and live:
            k = rng.choice(list(live))
            new = live[k] + rng.choice([1, 1, 2, 7, 16, 33])
            before = [m.num_free_pages(g) for g in range(2)]
            if m.reserve(m.get(k), new):
                live[k] = new
                m.release_passed(m.get(k), new)
            else:
                assert [m.num_free_pages(g) for g in range(2)] == before
        elif live:
            k = rng.choice(list(live))
            m.close(k)
            del live[k]
        m.check_invariants()
    for k in list(live):
        m.close(k)
    assert m.num_free_pages(0) == 13 and m.num_free_pages(1) == 10 and m.num_open() == 0
    m.check_invariants()
