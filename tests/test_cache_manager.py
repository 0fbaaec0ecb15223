"""The cache manager's books: no page lost, held twice or freed twice, under random orders."""

import random

import pytest

from llm_pipeline_b200.cache import CacheError, CacheManager, KVPagesSpec, PagePool, StateSpec


def manager(num_pages=16, page_size=4, max_requests=4, window=None, extra=None, max_tokens=256):
    specs = [(KVPagesSpec(2, 16, None), None), (KVPagesSpec(2, 16, None), None)]
    if window is not None:
        specs.append((KVPagesSpec(2, 16, window), None))
    if extra:
        specs.extend(extra)
    return CacheManager(specs, page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                        max_request_tokens=max_tokens, device=None)


def test_pool_is_lifo_and_strict():
    pool = PagePool(4)
    a = pool.alloc(3)
    assert a == [0, 1, 2] and pool.num_free == 1 and pool.alloc(2) is None and pool.num_free == 1
    pool.free([1])
    assert pool.alloc(1) == [1]                      # the page freed last is used again first
    with pytest.raises(CacheError, match="freed twice"):
        pool.free([3])
    with pytest.raises(CacheError, match="does not belong"):
        pool.free([9])
    pool.free([0, 1, 2])
    assert pool.num_free == 4 and pool.high_water == 3


def test_layers_with_the_same_need_share_a_group_and_windows_get_their_own():
    m = manager(window=8)
    assert len(m.groups) == 2
    assert m.groups[0].cache_ids == [0, 1] and m.groups[1].cache_ids == [2]
    assert m.group_of_cache == {0: 0, 1: 0, 2: 1}


def test_reserve_grows_block_tables_and_is_all_or_nothing():
    m = manager(num_pages=5, page_size=4)
    m.admit("a")
    assert m.reserve("a", 9) and m.block_table("a", 0) == [0, 1, 2]
    m.commit("a", 9)
    assert m.reserve("a", 10) and len(m.block_table("a", 0)) == 3     # same page
    m.admit("b")
    assert not m.reserve("b", 12)                                      # needs 3, 2 free: nothing taken
    assert m.block_table("b", 0) == [] and m.groups[0].pool.num_free == 2
    assert m.reserve("b", 8)
    m.check()
    m.free("a")
    assert m.reserve("b", 12) and m.block_table("b", 0)[-1] == 0       # a's pages are reused first, in the order a held them
    assert m.pages_reused == 1
    m.free("b")
    m.check()
    assert m.groups[0].pool.num_free == 5
    with pytest.raises(CacheError, match="not live"):
        m.free("b")


def test_token_slots_and_limits():
    m = manager(num_pages=8, page_size=4, max_tokens=20)
    m.admit("a")
    m.reserve("a", 6)
    assert [m.token_slot("a", 0, p) for p in range(6)] == [0, 1, 2, 3, 4, 5]
    assert not m.can_reserve("a", 21)
    with pytest.raises(CacheError, match="limit"):
        m.reserve("a", 21)


def test_window_group_gives_pages_back_while_the_request_lives():
    m = manager(num_pages=8, page_size=4, window=6)
    m.admit("a")
    assert m.reserve("a", 16)
    assert m.groups[1].pool.num_used == 4
    m.commit("a", 16)          # next query sits at 16 and sees keys 11..16: pages 0 and 1 are out of sight
    assert m.block_table("a", 1) == [-1, -1, 2, 3] and m.groups[1].pool.num_used == 2
    assert m.block_table("a", 0) == [0, 1, 2, 3]                       # the full-attention group keeps all
    assert m.token_slot("a", 1, 3) == -1
    assert m.reserve("a", 17)
    assert m.block_table("a", 1)[4] == 0                               # a page it gave back itself
    m.check()
    m.free("a")
    m.check()
    assert m.groups[1].pool.num_free == 8


def test_slots_are_reused_and_limited():
    m = manager(max_requests=2, extra=[(None, StateSpec((3,)))])
    s0, s1 = m.admit("a"), m.admit("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(CacheError, match="slots"):
        m.admit("c")
    with pytest.raises(CacheError, match="already live"):
        m.admit("a")
    m.free("a")
    assert m.admit("c") == s0
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page_size=4, max_requests=5, window=10 if seed % 2 else None)
    live = {}
    next_id = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            m.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            grow = rng.choice([1, 1, 1, 2, 5, 13])
            want = live[rid] + grow
            if m.can_reserve(rid, want):
                assert m.reserve(rid, want)
                m.commit(rid, want)
                live[rid] = want
            else:
                before = [g.pool.num_free for g in m.groups]
                if want <= m.max_request_tokens:
                    assert not m.reserve(rid, want)
                assert before == [g.pool.num_free for g in m.groups]
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        for rid, length in live.items():
            assert m.length(rid) == length
            full = m.block_table(rid, 0)
            assert len(full) == -(-length // 4) and all(p >= 0 for p in full)
    for rid in list(live):
        m.free(rid)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups)
    assert m.free_slots == 5


def test_admissions_are_numbered():
    """A request that ends and comes back under the same name is another admission: who remembers block tables by
    name can tell the two apart."""
    m = manager()
    m.admit("a")
    m.admit("b")
    first_a, first_b = m.admission("a"), m.admission("b")
    assert first_a != first_b
    m.free("a")
    m.admit("a")
    assert m.admission("a") not in (first_a, first_b) and m.admission("b") == first_b
    with pytest.raises(KeyError):
        m.admission("c")
