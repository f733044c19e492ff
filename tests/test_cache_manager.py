"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; handles go stale; reservations are all or
nothing.  The cases follow the reference's manager tests
(test/test_kv_cache_manager.cpp:80,114,148,165,449; test/test_sequence_kv_manager.cpp:24,60,96)."""
import random

import pytest

from paged_batch_engine_b200.cache import NO_PAGE, CacheError, CacheManager, KVGroupSpec


def full(layers=(0, 1)):
    return KVGroupSpec(tuple(layers), num_kv_heads=2, head_dim=16)


def windowed(w, layers=(2,)):
    return KVGroupSpec(tuple(layers), num_kv_heads=2, head_dim=16, window=w)


def test_pool_allocate_release_generation():
    m = CacheManager([full((0,))], page_tokens=1, num_pages=3, max_requests=4)
    pool = m.pools[0]
    hs = [m.add_request() for _ in range(3)]
    assert all(m.reserve(h, 1) for h in hs)
    pages = [m.block_table(h)[0] for h in hs]
    assert sorted(pages) == [0, 1, 2] and pool.num_free == 0
    extra = m.add_request()
    assert not m.reserve(extra, 1)                       # the pool is dry: nothing changes
    m.free(hs[1])
    assert pool.num_free == 1
    assert m.reserve(extra, 1)
    again = m.block_table(extra)[0]
    assert again == pages[1] and pool.generation[again] == 2       # used again, with a new generation
    assert pool.refcount(again) == 1 and pool.allocations == 4
    with pytest.raises(CacheError):
        m.free(hs[1])                                    # freed twice: the handle is stale
    m.check_invariants()


def test_append_across_page_edges_and_slots():
    m = CacheManager([full()], page_tokens=8, num_pages=4)
    h = m.add_request("r")
    assert m.reserve(h, 5) and len(m.block_table(h)) == 1
    m.commit(h, 5)
    assert m.reserve(h, 3) and len(m.block_table(h)) == 1          # fills the page exactly
    assert m.reserve(h, 1) and len(m.block_table(h)) == 2          # crosses the edge
    m.commit(h, 4)
    assert m.context_len(h) == 9 and m.reserved_len(h) == 9
    t = m.block_table(h)
    assert m.slot_of_token(h, 0, 7) == t[0] * 8 + 7 and m.slot_of_token(h, 0, 8) == t[1] * 8
    m.check_invariants()


def test_reservation_is_all_or_nothing_across_groups():
    m = CacheManager([full(), windowed(100)], page_tokens=4, num_pages=[8, 2])
    h = m.add_request()
    assert m.reserve(h, 8)                      # 2 pages in each group; group 1 is now full
    before = (m.num_free_pages(0), m.num_free_pages(1), m.reserved_len(h), list(m.block_table(h, 0)))
    assert not m.can_reserve(h, 1) and not m.reserve(h, 1)
    assert (m.num_free_pages(0), m.num_free_pages(1), m.reserved_len(h), list(m.block_table(h, 0))) == before
    assert m.pages_needed(h, 1) == [1, 1] and m.max_appendable_tokens(h) == 0
    m.check_invariants()


def test_free_gives_everything_back_and_handles_go_stale():
    m = CacheManager([full()], page_tokens=4, num_pages=6, max_requests=2)
    h1, h2 = m.add_request(), m.add_request()
    assert m.add_request() is None                           # no request slot left
    assert m.reserve(h1, 9) and m.reserve(h2, 4)
    assert m.num_free_pages() == 2
    slot = m.state_slot(h1)
    m.free(h1)
    assert m.num_free_pages() == 5 and not m.is_live(h1)
    for call in (lambda: m.context_len(h1), lambda: m.reserve(h1, 1), lambda: m.free(h1)):
        with pytest.raises(CacheError):
            call()
    h3 = m.add_request()
    assert m.state_slot(h3) == slot and h3 != h1            # same slot, new generation
    with pytest.raises(CacheError):
        m.block_table(-5)
    with pytest.raises(CacheError):
        m.block_table((1 << 40) | 77)
    m.check_invariants()


def test_many_lifetimes_reuse_one_slot():
    m = CacheManager([full()], page_tokens=4, num_pages=2, max_requests=1)
    seen = set()
    for i in range(2000):
        h = m.add_request()
        assert h not in seen
        seen.add(h)
        assert m.reserve(h, 5)
        m.commit(h, 5)
        m.free(h)
    assert m.num_free_pages() == 2
    m.check_invariants()


def test_commit_beyond_reservation_and_truncate():
    m = CacheManager([full()], page_tokens=4, num_pages=4)
    h = m.add_request()
    m.reserve(h, 10)
    with pytest.raises(CacheError):
        m.commit(h, 11)
    m.commit(h, 10)
    m.truncate(h, 5)
    assert m.context_len(h) == 5 and len(m.block_table(h)) == 2 and m.num_free_pages() == 2
    m.truncate(h, 0)
    assert m.num_free_pages() == 4
    m.check_invariants()


def test_window_gives_pages_back_when_passed():
    W, P = 6, 4
    m = CacheManager([full((0,)), windowed(W, (1,))], page_tokens=P, num_pages=[16, 16])
    h = m.add_request()
    held = []
    for n in range(1, 41):
        assert m.reserve(h, 1)
        m.commit(h, 1)
        table = m.block_table(h, 1)
        live = [b for b, p in enumerate(table) if p != NO_PAGE]
        # the next query (position n) reads keys n-W+1 .. n: their pages must all be held
        first_needed = max(0, n - W + 1)
        assert live and live[0] <= first_needed // P
        # nothing that lies wholly below the window is kept
        assert live[0] == first_needed // P
        held.append(len(live))
        assert all(p != NO_PAGE for p in m.block_table(h, 0))       # the full group keeps all
    assert max(held) <= (W + P - 1) // P + 1
    assert m.pools[1].allocations > m.pools[1].num_pages - m.num_free_pages(1)   # pages came back
    m.check_invariants()
    m.free(h)
    assert m.num_free_pages(1) == 16 and m.num_free_pages(0) == 16


def test_window_release_never_drops_a_needed_page_in_portions():
    W, P = 10, 4
    for portions in ([7, 2, 16, 3, 2, 9], [40], [1] * 30, [3, 30, 2, 2]):
        m = CacheManager([windowed(W, (0,))], page_tokens=P, num_pages=32)
        h = m.add_request()
        n = 0
        for c in portions:
            assert m.reserve(h, c)
            table = m.block_table(h, 0)
            # rows n .. n+c-1 read keys from n-W+1 on: those pages are held during the step
            for key in range(max(0, n - W + 1), n + c):
                assert table[key // P] != NO_PAGE
            m.commit(h, c)
            n += c
        m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    P = rng.choice([4, 8, 16])
    groups = [full((0, 1))] + ([windowed(rng.choice([5, 17]), (2,))] if seed % 2 else [])
    m = CacheManager(groups, page_tokens=P, num_pages=[rng.randint(6, 20) for _ in groups],
                     max_requests=5, lifo=bool(seed & 2))
    live = {}
    dead = []
    for step in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            h = m.add_request(step)
            assert h is not None and h not in live and h not in dead
            live[h] = 0
        elif op < 0.75 and live:
            h = rng.choice(list(live))
            n = rng.randint(1, 3 * P)
            free_before = [m.num_free_pages(g) for g in range(len(groups))]
            ok = m.reserve(h, n)
            if ok:
                m.commit(h, rng.randint(0, n) if rng.random() < 0.2 else n)
                if m.context_len(h) < m.reserved_len(h):
                    m.commit(h, m.reserved_len(h) - m.context_len(h))
                live[h] += n
                assert m.context_len(h) == live[h]
            else:
                assert free_before == [m.num_free_pages(g) for g in range(len(groups))]
        elif live:
            h = rng.choice(list(live))
            m.free(h)
            del live[h]
            dead.append(h)
            with pytest.raises(CacheError):
                m.free(h)
        m.check_invariants()
        # no page is in two live block tables
        for g in range(len(groups)):
            pages = [p for h in live for p in m.block_table(h, g) if p != NO_PAGE]
            assert len(pages) == len(set(pages))
    for h in list(live):
        m.free(h)
    assert all(m.num_free_pages(g) == m.pools[g].num_pages for g in range(len(groups)))


def test_state_slots_are_distinct_among_live_requests():
    m = CacheManager([], page_tokens=8, num_pages=[], max_requests=4)
    hs = [m.add_request() for _ in range(4)]
    assert sorted(m.state_slot(h) for h in hs) == [0, 1, 2, 3]
    assert m.reserve(hs[0], 1000) and m.max_appendable_tokens(hs[0]) > 1000   # no paged group: no limit
    m.commit(hs[0], 1000)
    m.free(hs[2])
    h = m.add_request()
    assert m.state_slot(h) == 2


def test_captured_step_split_capacity_covers_every_request_of_the_step():
    """The split capacity of a captured decode step is computed from the longest request
    alone; under a window a shorter request can touch one more split than the longest
    (window 512, splits of 256: 2,304 keys touch 2 splits, 1,704 keys touch 3).  The bound
    must hold for every shorter request, and the work-list fill must accept them all."""
    import numpy as np
    from paged_batch_engine_b200.cache.manager import decode_work_fill
    from paged_batch_engine_b200.engine.graphs import splits_bound
    rng = random.Random(7)
    cases = [(2304, 1704, 512, 256), (2304, 1704, 512, 512), (4096, 257, 300, 256), (1000, 999, None, 256)]
    for _ in range(400):
        sk = rng.choice([256, 512])
        W = rng.choice([None, 1, 2, 24, 150, 255, 256, 257, 511, 512, 513, 1000, 4096])
        longest = rng.randint(1, 6000)
        cases.append((longest, rng.randint(1, longest), W, sk))
    for longest, other, W, sk in cases:
        S = splits_bound(longest, W, sk)
        ctx = np.array([longest - 1, other - 1], dtype=np.int64)
        work = np.zeros((2 * S, 4), dtype=np.int32)
        counts = np.zeros(2, dtype=np.int32)
        worst = decode_work_fill(2, 2, S, ctx, W, sk, work, counts, None, None, None, None, refresh=True)
        assert 1 <= worst <= S, (longest, other, W, sk, S, worst)
        for r, n in enumerate((longest, other)):
            lo = max(0, n - W) if W else 0
            assert counts[r] == (n + sk - 1) // sk - lo // sk
    # the bound is tight somewhere: some shorter request does use all of it
    S = splits_bound(2304, 512, 256)
    assert S == 3


def test_page_directory_counts_owners_and_further_holds():
    """A page knows who it was handed to; a further hold keeps it out of the free queue after
    its request has given it back, and it returns when the last hold lets go."""
    m = CacheManager([full()], page_tokens=4, num_pages=6)
    a, b = m.add_request(), m.add_request()
    assert m.reserve(a, 9) and m.reserve(b, 4)
    ta, tb = m.block_table(a), m.block_table(b)
    assert [m.page_owner(0, p) for p in ta] == [a] * 3 and m.page_owner(0, tb[0]) == b
    free = [p for p in range(6) if p not in ta + tb]
    assert all(m.page_owner(0, p) is None for p in free)
    with pytest.raises(CacheError):
        m.share_page(0, free[0])                      # a free page cannot be shared
    m.share_page(0, ta[1])
    m.share_page(0, ta[1])
    assert m.pools[0].refcount(ta[1]) == 3
    m.check_invariants()
    m.free(a)
    assert m.num_free_pages() == 6 - 1 - 1            # b's page and the shared one are still out
    assert m.pools[0].refcount(ta[1]) == 2 and m.page_owner(0, ta[1]) == a
    m.check_invariants()
    m.unshare_page(0, ta[1])
    m.unshare_page(0, ta[1])
    assert m.num_free_pages() == 5 and m.page_owner(0, ta[1]) is None
    with pytest.raises(CacheError):
        m.unshare_page(0, ta[1])
    m.check_invariants()


def test_reset_gives_everything_back_and_stales_the_handles():
    m = CacheManager([full((0,)), windowed(6, (1,))], page_tokens=4, num_pages=[8, 8])
    hs = [m.add_request() for _ in range(3)]
    for i, h in enumerate(hs):
        assert m.reserve(h, 5 + 3 * i)
        m.commit(h, 5 + 3 * i)
    assert sorted(m.live_handles()) == sorted(hs)
    m.reset()
    assert m.num_live_requests == 0 and m.num_free_pages(0) == 8 and m.num_free_pages(1) == 8
    assert not any(m.is_live(h) for h in hs)
    m.check_invariants()
    h = m.add_request()
    assert m.reserve(h, 32) and h not in hs
