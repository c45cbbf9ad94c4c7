"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; window groups give pages back; state slots."""
import random

import pytest

from qwen_decoder_b200.cache import (BlockTable, CacheAccountingError, CacheLayout, CacheManager, FixedState,
                                     OutOfPages, PagedKV, PagePool, StateSlots)


def test_pool_order_and_errors():
    p = PagePool(3)
    a, b, c = p.allocate(), p.allocate(), p.allocate()
    assert (a, b, c) == (0, 1, 2) and p.num_free == 0
    with pytest.raises(OutOfPages):
        p.allocate()
    p.release(b)
    p.release(a)
    with pytest.raises(CacheAccountingError):
        p.release(a)                       # freed twice
    with pytest.raises(CacheAccountingError):
        p.retain(a)                        # retain of a free page
    assert p.allocate() == b               # the page freed longest ago comes back first
    p.retain(c)
    p.release(c)
    assert p.ref_count(c) == 1 and p.num_free == 1
    p.check()


def test_state_slots():
    s = StateSlots(2)
    a, b = s.allocate(), s.allocate()
    with pytest.raises(OutOfPages):
        s.allocate()
    s.release(a)
    with pytest.raises(CacheAccountingError):
        s.release(a)
    assert s.allocate() == a


def layout(window=None, extra_fixed=False):
    needs = [PagedKV(2, 16), PagedKV(2, 16, window), PagedKV(2, 16)]
    if extra_fixed:
        needs.append(FixedState((4,)))
    return CacheLayout.from_needs(needs, [None] * len(needs))


def test_layout_groups_layers_by_need():
    lo = layout(window=None)
    assert len(lo.groups) == 1 and lo.paged == {0: (0, 0), 1: (0, 1), 2: (0, 2)}
    lo = layout(window=40, extra_fixed=True)
    assert len(lo.groups) == 2 and lo.paged[1] == (1, 0) and lo.paged[2] == (0, 1) and lo.fixed == {3: 0}
    # a run that reads another run's cache maps to the same place and owns nothing
    lo = CacheLayout.from_needs([PagedKV(1, 8), PagedKV(1, 8), PagedKV(1, 8)], [None, 0, None])
    assert lo.paged == {0: (0, 0), 1: (0, 0), 2: (0, 1)} and lo.groups[0].entries == [0, 2]
    with pytest.raises(ValueError):
        CacheLayout.from_needs([PagedKV(1, 8), PagedKV(2, 8)], [None, 0])


def test_ensure_is_all_or_nothing_and_close_frees():
    m = CacheManager(layout(window=None), num_pages=4, page_size=16, max_requests=4)
    a = m.open("a")
    m.ensure(a, 33)
    assert len(a.tables[0]) == 3 and m.free_pages() == [1]
    b = m.open("b")
    with pytest.raises(OutOfPages):
        m.ensure(b, 17)
    assert len(b.tables[0]) == 0 and m.free_pages() == [1]
    m.commit(a, 33)
    with pytest.raises(CacheAccountingError):
        m.commit(a, 16)                    # more tokens than pages
    m.close(a)
    with pytest.raises(CacheAccountingError):
        m.close(a)
    m.close(b)
    m.check()
    assert m.free_pages() == [4] and m.slots.num_free == 4


def test_window_group_gives_pages_back():
    m = CacheManager(layout(window=40), num_pages=8, page_size=16, max_requests=2)
    r = m.open("r")
    total = 0
    for n in [30, 1, 1, 20, 1, 40, 1]:
        m.ensure(r, total + n)
        m.commit(r, n)
        total += n
        full, win = r.tables
        assert len(full.live_pages()) == (total + 15) // 16
        first_needed = max(0, total - 40 + 1) // 16
        assert win.first_live == first_needed
        assert win.pages[:first_needed] == [BlockTable.RELEASED] * first_needed
        assert len(win.live_pages()) == (total + 15) // 16 - first_needed
        m.check()
    m.close(r)
    assert m.free_pages() == [8, 8]


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = CacheManager(layout(window=24, extra_fixed=True), num_pages=12, page_size=8, max_requests=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            n = rng.choice([1, 1, 1, 2, 7, 19])
            try:
                m.ensure(rc, rc.num_tokens + n)
                m.commit(rc, n)
            except OutOfPages:
                victim = rng.choice(list(live))
                m.close(live.pop(victim))
        elif live:
            m.close(live.pop(rng.choice(list(live))))
        m.check()
        for g, pool in enumerate(m.pools):
            named = sum(len(rc.tables[g].live_pages()) for rc in live.values())
            assert pool.num_used == named
        assert m.slots.num_free == 4 - len(live)
    for rc in list(live.values()):
        m.close(rc)
    assert m.free_pages() == [12, 12]
