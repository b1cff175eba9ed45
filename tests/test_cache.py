"""The cache manager on the host: pools, groups, block tables, windows, slots; no page is
lost, held twice or freed twice under random orders of requests."""

import random

import pytest

from qwen25vl_lite.cache import CacheManager, NoFreeSlot, OutOfPages, PagePool, StopNeeds
from qwen25vl_lite.parts import KVCacheNeed, StateNeed


def test_pool_is_strict():
    pool = PagePool(4)
    a = pool.allocate(3)
    assert a == [3, 2, 1] and pool.num_free == 1 and pool.in_use() == 3      # handed out from the top (LIFO)
    with pytest.raises(OutOfPages):
        pool.allocate(2)
    assert pool.num_free == 1                                                # all-or-nothing
    pool.free([2])
    assert pool.allocate(1) == [2]                                           # a page given back is used again first
    with pytest.raises(ValueError, match="outside"):
        pool.free([9])
    with pytest.raises(ValueError, match="not held"):
        pool.free([0])
    pool.free([1])
    with pytest.raises(ValueError, match="not held"):
        pool.free([1])                                                       # double free
    pool.fork([3])
    pool.free([3])
    assert pool.refcount(3) == 1 and pool.in_use() == 2
    pool.check()


def _manager(pages=16, page=4, slots=3):
    full, win = KVCacheNeed(2, 16, None), KVCacheNeed(2, 16, 10)
    stops = [StopNeeds(win), StopNeeds(full), StopNeeds(win), StopNeeds(full, cache_of=1), StopNeeds(None, StateNeed((3,)))]
    return CacheManager(stops, pages, page, slots)


def test_groups_and_locations():
    m = _manager()
    assert [g.window for g in m.groups] == [10, None]
    assert m.groups[0].stops == [0, 2] and m.groups[1].stops == [1]
    assert m.location[3] == m.location[1]                 # a stop that reads another stop's cache
    assert 4 in m.state_needs and 4 not in m.location
    with pytest.raises(ValueError, match="keeps none"):
        CacheManager([StopNeeds(None), StopNeeds(KVCacheNeed(1, 16), cache_of=0)], 4, 4, 1)
    with pytest.raises(ValueError, match="shapes differ"):
        CacheManager([StopNeeds(KVCacheNeed(1, 16)), StopNeeds(KVCacheNeed(2, 16), cache_of=0)], 4, 4, 1)
    with pytest.raises(ValueError, match="window"):
        CacheManager([StopNeeds(KVCacheNeed(1, 16, 8)), StopNeeds(KVCacheNeed(1, 16, None), cache_of=0)], 4, 4, 1)


def test_block_tables_grow_and_windows_give_pages_back():
    m = _manager()
    r = m.open()
    m.ensure(r, 9)                                        # 9 tokens: 3 pages in each group
    assert [len(t) for t in r.tables] == [3, 3] and m.pages_in_use() == [3, 3]
    m.ensure(r, 9)
    assert m.pages_in_use() == [3, 3]                     # idempotent
    m.advance(r, 9)
    assert m.pages_in_use() == [3, 3]                     # token 9 still sees keys 0..9 (window 10)
    m.ensure(r, 14)
    m.advance(r, 5)                                       # 14 tokens in: next token sees keys 5..14 -> page 0 is behind
    assert r.tables[0][0] == -1 and m.pages_in_use() == [3, 4]
    m.ensure(r, 30)
    m.advance(r, 16)                                      # next token (30) sees keys 21..30: pages 0..4 are behind
    assert [p >= 0 for p in r.tables[0]] == [False] * 5 + [True] * 3
    assert m.pages_in_use() == [3, 8]
    m.check([r])
    m.close(r)
    assert m.pages_in_use() == [0, 0] and m.free_slots == 3
    with pytest.raises(ValueError, match="already closed"):
        m.close(r)


def test_all_or_nothing_across_groups():
    m = _manager(pages=4)
    a, b = m.open(), m.open()
    m.ensure(a, 12)                                       # 3 of 4 pages in both groups
    with pytest.raises(OutOfPages):
        m.ensure(b, 8)
    assert m.pages_in_use() == [3, 3] and b.tables == [[], []]
    assert not m.can_hold(b, 8) and m.can_hold(b, 4)
    m.check([a, b])


def test_slots():
    m = _manager(slots=2)
    a, b = m.open(), m.open()
    assert {a.slot, b.slot} == {0, 1}
    with pytest.raises(NoFreeSlot):
        m.open()
    m.close(a)
    c = m.open()
    assert c.slot == a.slot and c.num_tokens == 0 and c.position_offset == 0


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    m = _manager(pages=24, page=4, slots=5)
    live = []
    grown = freed = 0
    for _ in range(600):
        roll = rng.random()
        if roll < 0.15 and m.free_slots:
            live.append(m.open())
        elif roll < 0.8 and live:
            r = rng.choice(live)
            n = rng.randint(1, 13)
            try:
                m.ensure(r, r.num_tokens + n)
                m.advance(r, n)
                grown += 1
            except OutOfPages:
                victim = rng.choice(live)
                m.close(victim)
                live.remove(victim)
                freed += 1
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.close(r)
            freed += 1
        m.check(live)
        for r in live:                                    # every key the next token sees has a page
            for g in m.groups:
                first = g.first_needed_page(r.num_tokens)
                assert all(p >= 0 for p in r.tables[g.index][first:-(-r.num_tokens // 4)])
    for r in live:
        m.close(r)
    m.check([])
    assert m.pages_in_use() == [0, 0] and m.free_slots == 5 and grown > 100 and freed > 10
