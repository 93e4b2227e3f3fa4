"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest

from oxr_inference_b200.cache import RELEASED, CacheManager, PagePool, make_cache_plan, pages_for
from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed


def _plan(windows=(0,), states=0):
    needs = [PagedKVNeed(2, 16, w) for w in windows] + [StateNeed((4,)) for _ in range(states)]
    return make_cache_plan(needs, [None] * len(needs))


def test_pool_is_lifo_page_zero_first_and_all_or_nothing():
    pool = PagePool(4)
    assert pool.allocate(2) == [0, 1] and pool.allocate(3) is None and pool.free == 2
    pool.release([0, 1])
    assert pool.allocate(2) == [0, 1], "pages given back are handed out again at once"
    with pytest.raises(ValueError, match="twice"):
        pool.release([3])
    with pytest.raises(ValueError, match="not of this pool"):
        pool.release([4])


def test_layers_with_the_same_need_share_a_group_others_get_their_own():
    needs = [PagedKVNeed(2, 16, 0), PagedKVNeed(2, 16, 24), PagedKVNeed(2, 16, 0), StateNeed((3, 5)), None, PagedKVNeed(2, 16, 0)]
    plan = make_cache_plan(needs, [None, None, None, None, None, 0])
    assert [g.num_layers for g in plan.groups] == [2, 1] and plan.groups[1].need.window == 24
    e = plan.entries
    assert (e[0].group, e[0].layer_in_group, e[2].group, e[2].layer_in_group, e[1].group) == (0, 0, 0, 1, 1)
    assert e[3].state == 0 and e[3].group is None and e[4].group is None and e[4].state is None
    assert (e[5].group, e[5].layer_in_group, e[5].store) == (0, 0, False), "entry 5 reads entry 0's cache"
    with pytest.raises(ValueError, match="later entry"):
        make_cache_plan(needs[:2] + needs[:1], [2, None, None])
    with pytest.raises(ValueError, match="none of its own"):
        make_cache_plan([needs[0], needs[0], needs[0]], [None, 0, 1])
    with pytest.raises(ValueError, match="but reads the cache"):
        make_cache_plan(needs[:2], [None, 0])


def test_reserve_advance_close_and_slots():
    m = CacheManager(_plan(), page_size=8, num_pages=6, max_requests=2)
    assert m.usable_pages == 5 and m.free_pages == 5 and m.scratch_pages == [0]
    a = m.open("a")
    assert m.reserve(a, 17) and a.tables == [[1, 2, 3]] and m.free_pages == 2
    assert m.slots(a, 0, 6, 10).tolist() == [14, 15, 16, 17]
    m.advance(a, 17)
    assert m.reserve(a, 24) and a.tables == [[1, 2, 3]], "room was there already"
    b = m.open("b")
    assert not m.reserve(b, 17) and b.tables == [[]] and m.free_pages == 2, "all or nothing"
    assert m.open("c") is None, "no third state slot"
    with pytest.raises(ValueError, match="beyond"):
        m.advance(b, 5)
    m.close(a)
    assert m.reserve(b, 17) and b.tables == [[1, 2, 3]], "b gets a's pages"
    with pytest.raises(ValueError, match="twice"):
        m.close(a)
    m.close(b)
    m.check()
    assert m.free_pages == 5 and m.free_slots == 2


def test_a_window_gives_pages_back_as_it_passes_them():
    m = CacheManager(_plan(windows=(0, 20)), page_size=8, num_pages=12, max_requests=2)
    r = m.open()
    assert m.reserve(r, 50)
    m.advance(r, 50)  # next query at 50 sees keys 31..50 -> pages 0..2 (positions 0..23) are behind the window
    assert r.tables[0] == [1, 2, 3, 4, 5, 6, 7] and r.tables[1][:3] == [RELEASED] * 3 and r.tables[1][3:] == [4, 5, 6, 7]
    assert m.pools[1].free == 11 - 4 and m.pools[0].free == 11 - 7
    with pytest.raises(ValueError, match="released"):
        m.slots(r, 1, 20, 30)
    assert m.reserve(r, 60)
    assert r.tables[1][7] in (1, 2, 3), "a page the window released is used again"
    m.advance(r, 60)
    m.check()
    m.close(r)
    m.check()
    assert m.free_pages == 11


def test_bytes_per_page():
    import torch

    plan = make_cache_plan([PagedKVNeed(8, 128, 0)] * 36, [None] * 36)
    assert CacheManager.bytes_per_page(plan, 16, torch.bfloat16) == 2 * 36 * 16 * 8 * 128 * 2  # oxr_runtime/kv_cache.py:34-37
    assert pages_for(0, 16) == 0 and pages_for(1, 16) == 1 and pages_for(16, 16) == 1 and pages_for(17, 16) == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_never_lose_or_double_a_page(seed):
    rng = random.Random(seed)
    windows = [(0,), (0, 12), (7, 0, 30)][seed % 3]
    m = CacheManager(_plan(windows, states=1), page_size=4, num_pages=40, max_requests=5)
    live = []
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            rc = m.open(rng.random())
            assert rc is not None
            live.append(rc)
        elif action < 0.85 and live:
            rc = rng.choice(live)
            new = rc.length + rng.choice([1, 1, 1, 2, 5, 17, 40])
            before = [list(t) for t in rc.tables]
            if m.reserve(rc, new):
                # positions to be written all lie on live pages, no page of this request is shared with another
                for g in range(len(m.pools)):
                    slots = m.slots(rc, g, rc.length, new)
                    assert len(set(slots.tolist())) == new - rc.length
                if rng.random() < 0.9:
                    m.advance(rc, new)
            else:
                assert rc.tables == before, "a failed reserve must take nothing"
        elif live:
            rc = live.pop(rng.randrange(len(live)))
            m.close(rc)
        m.check()
        held = [p for rc in live for p in rc.tables[0] if p != RELEASED]
        assert len(held) == len(set(held))
    for rc in live:
        m.close(rc)
    m.check()
    assert all(p.free == 39 for p in m.pools) and m.free_slots == 5


def test_window_never_releases_a_page_a_later_query_needs():
    """Brute force: after any sequence of advances, every key inside the window of the next query is on a live page."""
    rng = random.Random(3)
    for window in (1, 5, 8, 13):
        m = CacheManager(_plan((window,)), page_size=4, num_pages=64, max_requests=1)
        rc = m.open()
        length = 0
        while length < 120:
            step = rng.choice([1, 2, 3, 9, 20])
            assert m.reserve(rc, length + step)
            # during the step the first new query (position `length`) must still see its window
            for key in range(max(0, length - window + 1), length + step):
                assert rc.tables[0][key // 4] != RELEASED
            length += step
            m.advance(rc, length)
            live_pages = sum(p != RELEASED for p in rc.tables[0])
            assert live_pages <= (window + 3) // 4 + 2, "pages behind the window must have been given back"
        m.close(rc)


def test_a_request_is_named_by_a_serial_that_is_never_given_twice():
    """Copies of block-table rows are remembered by (serial, version). ``id()`` would not do: a closed request's
    address goes to a later request, whose version numbers run through the same values."""
    m = CacheManager(_plan(windows=(0, 12)), page_size=8, num_pages=8, max_requests=2)
    seen = set()
    for _ in range(50):
        rc = m.open()
        assert rc.serial not in seen
        seen.add(rc.serial)
        assert m.reserve(rc, 20)
        m.advance(rc, 20)
        m.close(rc)
        del rc


def test_room_is_what_the_held_pages_can_take():
    """``room`` lets reserve and advance answer with one comparison; it follows the shortest table."""
    m = CacheManager(_plan(windows=(0, 12)), page_size=8, num_pages=10, max_requests=2)
    r = m.open("a")
    assert r.room == 0 and r.released == [0, 0]
    assert m.reserve(r, 9) and r.room == 16 and [len(t) for t in r.tables] == [2, 2]
    version = r.version
    assert m.reserve(r, 16) and r.version == version          # nothing new was needed
    with pytest.raises(ValueError):
        m.advance(r, 17)                                       # beyond what was reserved
    m.advance(r, 16)
    assert m.reserve(r, 40) and r.room == 40
    m.advance(r, 40)                                           # the window of 12 has passed positions 0..28: pages 0..2
    assert r.released == [0, 3] and r.tables[1][:3] == [RELEASED] * 3 and r.room == 40
    m.check()
    m.close(r)
    assert r.room == 0 and r.released == [0, 0]
    m.check()
