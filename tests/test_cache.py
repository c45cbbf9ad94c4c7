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


# ------------------------------------------------------------------ prefix cache
def prefix_manager(num_pages=12, page_size=4, groups=1):
    needs = [PagedKV(2, 16)] + ([PagedKV(1, 8)] if groups == 2 else [])
    lo = CacheLayout.from_needs(needs, [None] * len(needs))
    return CacheManager(lo, num_pages, page_size, max_requests=4, prefix_cache=True)


def feed(m, rc, tokens):
    m.ensure(rc, rc.num_tokens + len(tokens))
    m.commit(rc, len(tokens), tokens)


def test_prefix_pages_are_shared_exactly_and_leave_one_token():
    m = prefix_manager(groups=2)
    a = m.open("a", list(range(100, 111)))           # 11 tokens: nothing cached yet
    assert a.num_tokens == 0
    feed(m, a, list(range(100, 111)))                # pages 0 and 1 are full and recorded
    b = m.open("b", list(range(100, 108)) + [7, 7, 7])
    assert b.num_tokens == 8 and [t.pages[:2] for t in b.tables] == [t.pages[:2] for t in a.tables]
    assert all(m.pools[g].ref_count(a.tables[g].pages[0]) == 2 for g in range(2))
    c = m.open("c", list(range(100, 108)))           # all 8 tokens known: one page stays to be computed
    assert c.num_tokens == 4
    d = m.open("d", [100, 101, 102, 999] + list(range(104, 111)))   # differs inside the first page: no hit
    assert d.num_tokens == 0
    m.check()
    for rc in (a, b, c, d):
        m.close(rc)
    m.check()
    assert m.free_pages() == [12, 12]


def test_freed_pages_stay_cached_until_they_are_handed_out_again():
    m = prefix_manager(num_pages=4, page_size=4)
    a = m.open("a", None)
    feed(m, a, list(range(8)))                       # two full pages
    pages = list(a.tables[0].pages)
    m.close(a)
    assert m.free_pages() == [4]
    b = m.open("b", list(range(8)) + [50])           # hit on pages nobody holds: taken back off the free list
    assert b.num_tokens == 8 and b.tables[0].pages == pages and m.free_pages() == [2]
    m.close(b)
    c = m.open("c", None)
    feed(m, c, [9] * 16)                             # needs all four pages: the cached ones are overwritten
    m.close(c)
    d = m.open("d", list(range(8)) + [50])
    assert d.num_tokens == 0 and not any(k[1] == (0, 1, 2, 3) for k in m.prefix.children)
    m.close(d)
    m.check()


def test_prefix_cache_is_off_for_windows_and_state():
    lo = CacheLayout.from_needs([PagedKV(2, 16, 8)], [None])
    assert CacheManager(lo, 4, 4, 2, prefix_cache=True).prefix is None
    lo = CacheLayout.from_needs([PagedKV(2, 16), FixedState((3,))], [None, None])
    assert CacheManager(lo, 4, 4, 2, prefix_cache=True).prefix is None


@pytest.mark.parametrize("seed", range(4))
def test_prefix_cache_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = prefix_manager(num_pages=10, page_size=4, groups=2)
    stems = [[rng.randrange(5) for _ in range(12)] for _ in range(3)]
    live = {}
    for step in range(500):
        op = rng.random()
        if op < 0.3 and len(live) < 4:
            toks = rng.choice(stems)[:rng.choice([4, 8, 12])] + [rng.randrange(5) for _ in range(rng.randrange(1, 6))]
            try:
                rc = m.open(step, toks)
            except OutOfPages:
                continue
            assert rc.num_tokens % 4 == 0 and rc.num_tokens < len(toks) and rc.token_log == toks[:rc.num_tokens]
            live[step] = (rc, toks)
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            rc, toks = live[rid]
            n = rng.choice([1, 2, 5])
            new = toks[rc.num_tokens:rc.num_tokens + n] or [rng.randrange(5)]
            try:
                feed(m, rc, new)
                if rc.num_tokens > len(toks):
                    toks.extend(new[len(new) - (rc.num_tokens - len(toks)):])
            except OutOfPages:
                m.close(live.pop(rid)[0])
        elif live:
            m.close(live.pop(rng.choice(list(live)))[0])
        m.check()
        # every recorded entry points at pages whose books agree: held by someone or on the free list
        for e in m.prefix.entries.values():
            for g, p in enumerate(e.pages):
                assert m.prefix._by_page[g][p] in m.prefix.entries
    for rc, _ in list(live.values()):
        m.close(rc)
    assert m.free_pages() == [10, 10]
