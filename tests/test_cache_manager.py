"""The cache manager on the host: no page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from binfer_b200.cache import CacheManager, KVNeed, OutOfPages, PagePool, SlotPool, StateNeed


def _mgr(pages=8, page_size=4, window=None, max_requests=4):
    needs = [KVNeed(2, 16), KVNeed(2, 16, window) if window else KVNeed(2, 16), None]
    return CacheManager(needs, [None, None, StateNeed((3,))], page_size=page_size,
                        num_pages=pages, max_requests=max_requests)


def test_page_pool_reuses_last_freed_first_and_never_hands_out_page_zero():
    pool = PagePool(3)
    a, b, c = pool.alloc(), pool.alloc(), pool.alloc()
    assert sorted([a, b, c]) == [1, 2, 3]
    with pytest.raises(OutOfPages):
        pool.alloc()
    pool.free(b)
    assert pool.alloc() == b
    pool.free(a)
    with pytest.raises(ValueError, match="freed twice"):
        pool.free(a)
    with pytest.raises(ValueError):
        pool.free(0)
    with pytest.raises(ValueError):
        pool.free(4)


def test_slot_pool():
    s = SlotPool(2)
    a, b = s.alloc(), s.alloc()
    with pytest.raises(OutOfPages):
        s.alloc()
    s.free(a)
    with pytest.raises(ValueError):
        s.free(a)
    assert s.alloc() == a


def test_groups_by_geometry_and_window():
    m = _mgr(window=8)
    assert len(m.groups) == 2
    assert m.entry_location == [(0, 0), (1, 0), None]
    same = _mgr()
    assert len(same.groups) == 1 and same.entry_location == [(0, 0), (0, 1), None]


def test_reserve_is_all_or_nothing():
    m = _mgr(pages=4, page_size=4)
    m.add_request("a")
    m.reserve("a", 9)                       # 3 pages
    m.commit("a", 9)
    m.add_request("b")
    before = (m.num_free_pages(), [list(t) for t in m.get("b").tables])
    assert not m.can_reserve([("b", 8)])
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)                   # needs 2, only 1 free
    assert (m.num_free_pages(), [list(t) for t in m.get("b").tables]) == before
    m.reserve("b", 4)
    m.check_consistent()
    assert m.num_free_pages() == [0]
    assert m.can_reserve([("a", 12)]) and not m.can_reserve([("a", 13)])


def test_free_gives_everything_back_and_rejects_unknown():
    m = _mgr()
    m.add_request(1)
    m.reserve(1, 20)
    m.commit(1, 20)
    slot = m.get(1).slot
    m.free_request(1)
    assert m.num_free_pages() == [8] and m.slots.num_free == 4
    with pytest.raises(KeyError):
        m.free_request(1)
    m.add_request(2)
    assert m.get(2).slot == slot and m.get(2).fresh
    with pytest.raises(ValueError, match="already live"):
        m.add_request(2)


def test_window_pages_are_given_back_as_the_window_passes():
    m = _mgr(pages=6, page_size=4, window=8)
    m.add_request("r")
    full, win = m.groups
    for new_len in range(1, 41):            # token by token
        if new_len > 24:
            # the full-attention group is exhausted at 24 tokens; the windowed one goes on
            with pytest.raises(OutOfPages):
                m.reserve("r", new_len)
            break
        m.reserve("r", new_len)
        m.commit("r", new_len)
        m.check_consistent()
        held = [p for p in m.get("r").tables[1] if p > 0]
        assert len(held) <= 3               # window 8 over pages of 4: at most 3 pages live
    t = m.get("r").tables[1]
    # query at position 24 reads keys 17..24: pages 0..3 are passed
    m.release_passed("r")
    assert t[:4] == [-1, -1, -1, -1] and all(p > 0 for p in t[4:])
    m.free_request("r")
    assert m.num_free_pages() == [6, 6]


def test_window_first_needed_page():
    m = _mgr(page_size=4, window=8)
    g = m.groups[1]
    assert [g.first_needed_page(n) for n in (0, 7, 8, 11, 12)] == [0, 0, 0, 1, 1]
    assert m.groups[0].first_needed_page(1000) == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 6, 13])
    m = _mgr(pages=rng.randint(6, 20), page_size=rng.choice([1, 3, 4, 16]), window=window,
             max_requests=5)
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"q{step}"
            m.add_request(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.randint(1, 9)
            try:
                m.reserve(rid, new_len)
            except OutOfPages:
                assert not m.can_reserve([(rid, new_len)])
            else:
                m.commit(rid, new_len)
                live[rid] = new_len
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        m.check_consistent()
    for rid in list(live):
        m.free_request(rid)
    assert m.num_free_pages() == [g.pool.num_pages for g in m.groups]
    assert m.slots.num_free == 5


def test_groups_get_pools_of_their_own_size():
    """A windowed group keeps a window's worth of keys per request, so its pool is planned
    smaller than the pool of a group that keeps every key; the bytes it saves buy the other
    group more pages."""
    from binfer_b200.cache.manager import plan_pages
    full, win = KVNeed(2, 16), KVNeed(2, 16, window=32)
    needs = [full, win, win, full]
    page = 2 * 2 * 16 * 8 * 4                       # one page of one layer, float32
    budget = 40 * page * 4                          # 40 pages for every layer, were all alike
    pages = plan_pages(needs, page_size=8, budget_bytes=budget, element_size=4, max_requests=4,
                       max_seq_len=256, max_tokens_per_step=16)
    n_full, n_win = pages(full), pages(win)
    assert n_win < n_full and n_full > 40
    assert 2 * page * (n_full + n_win) <= budget
    # never more than the requests can use
    roomy = plan_pages(needs, 8, 10 ** 12, 4, max_requests=4, max_seq_len=256,
                       max_tokens_per_step=16)
    assert roomy(full) == 4 * (256 // 8 + 2) and roomy(win) == 4 * ((32 + 16) // 8 + 2)
    cm = CacheManager(needs, page_size=8, num_pages=pages, max_requests=4)
    assert [g.pool.num_pages for g in cm.groups] == [n_full, n_win]
    assert cm.num_pages == n_full
    # a long lone request fits if the full group can hold it; the windowed group only needs
    # its window (and the page being written)
    assert cm.can_ever_hold(n_full * 8) and not cm.can_ever_hold(n_full * 8 + 1)
    small = CacheManager([win], page_size=8, num_pages=4, max_requests=2)
    assert not small.can_ever_hold(1000)            # window 32 -> 5 pages + 1
    assert CacheManager([win], page_size=8, num_pages=6, max_requests=2).can_ever_hold(1000)


def test_a_windowed_request_runs_through_a_small_pool():
    """Far more tokens than the pool holds pass through a windowed group, portion by portion,
    because pages behind the window come back before a step takes new ones."""
    cm = CacheManager([KVNeed(1, 8, window=20)], page_size=4, num_pages=9, max_requests=1)
    cm.add_request("r")
    n = 0
    for step in range(60):
        n += 7
        assert cm.can_reserve([("r", n)])
        cm.reserve("r", n)
        cm.commit("r", n)
        cm.check_consistent()
    cm.free_request("r")
    assert cm.groups[0].pool.num_held == 0


def test_pages_of_a_tile_are_neighbours_where_the_pool_allows():
    """Two requests that grow in turn, a page at a time: with 16-token pages a 128-key tile
    is eight pages, and each request's eight lie side by side in the pool, because a request
    starts a tile in a run of pages that is wholly free and then takes the page behind its
    last one.  When no such page is left, it takes any: nothing is ever refused."""
    cm = CacheManager([KVNeed(1, 8)], page_size=16, num_pages=40, max_requests=4)
    for rid in "ab":
        cm.add_request(rid)
    for n in range(1, 17):                     # 16 pages each, in turn
        for rid in "ab":
            cm.reserve(rid, 16 * n)
            cm.commit(rid, 16 * n)
    for rid in "ab":
        t = cm.get(rid).tables[0]
        for tile in (t[:8], t[8:]):
            assert tile == list(range(tile[0], tile[0] + 8)), (rid, t)
    cm.check_consistent()
    # 8 pages are left, one whole run: c takes it, d finds only scattered pages later
    cm.add_request("c")
    cm.reserve("c", 16 * 8)
    assert cm.num_free_pages() == [0]
    cm.free_request("a")
    cm.add_request("d")
    cm.reserve("d", 16 * 16)                   # a's pages, whatever their order
    assert cm.num_free_pages() == [0]
    cm.check_consistent()
    for rid in "bcd":
        cm.free_request(rid)
    assert cm.groups[0].pool.num_held == 0


def test_page_pool_with_runs_never_loses_a_page():
    import random
    from binfer_b200.cache.pages import PagePool
    rng = random.Random(5)
    pool = PagePool(37, run=8)
    held = []
    for _ in range(20000):
        if held and (rng.random() < 0.5 or pool.num_free == 0):
            pool.free(held.pop(rng.randrange(len(held))))
        else:
            after = rng.choice(held) if held and rng.random() < 0.7 else 0
            p = pool.alloc(after=after, index=rng.randrange(20))
            assert p not in held and 1 <= p <= 37
            held.append(p)
        assert pool.num_free == 37 - len(held)
    while pool.num_free:                        # every free page can still be had
        held.append(pool.alloc())
    assert sorted(held) == list(range(1, 38))
