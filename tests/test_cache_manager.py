"""The cache manager's bookkeeping, without a GPU: no page is lost, held twice or freed
twice, under random orders of requests; windows give pages back; slots are exclusive."""
import random

import pytest

from flyweight_b200.cache import PAGE_SIZE, CacheManager, OutOfPages, OutOfSlots, PagePool
from flyweight_b200.parts import FixedState, PagedKV


def manager(num_pages=8, num_slots=4, window=None):
    specs = [PagedKV(2, 16), FixedState((8, 2)), PagedKV(2, 16), None]
    if window:
        specs.append(PagedKV(1, 32, window=window))
    return CacheManager(specs, num_pages, num_slots, device=None)


def test_pool_is_lifo_and_refuses_double_release():
    pool = PagePool(3)
    a, b = pool.allocate(), pool.allocate()
    assert (a, b) == (0, 1)
    pool.release(a)
    assert pool.allocate() == a                 # last freed, first reused
    pool.release(b)
    with pytest.raises(RuntimeError, match="not held"):
        pool.release(b)
    with pytest.raises(RuntimeError, match="not held"):
        pool.release(7)
    pool.allocate(), pool.allocate()
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.check()
    assert pool.high_water == 3


def test_layers_with_the_same_need_share_a_group():
    m = manager(window=100)
    assert len(m.groups) == 2
    assert m.groups[0].members == [0, 2] and m.groups[0].window == 0
    assert m.groups[1].members == [4] and m.groups[1].window == 100
    assert m.layer_caches[0].group == 0 and m.layer_caches[4].group == 1
    assert m.layer_caches[1].group is None and m.layer_caches[3].spec is None


def test_tables_grow_one_page_at_a_page_edge():
    m = manager()
    m.admit("r")
    m.extend("r", 1)
    assert len(m.groups[0].tables["r"]) == 1
    m.extend("r", PAGE_SIZE)
    assert len(m.groups[0].tables["r"]) == 1
    m.extend("r", PAGE_SIZE + 1)
    assert len(m.groups[0].tables["r"]) == 2
    assert m.block_table(0, ["r"], 4) == [m.groups[0].tables["r"] + [-1, -1]]
    with pytest.raises(ValueError, match="never shrinks"):
        m.extend("r", 3)
    m.check()


def test_out_of_pages_changes_nothing():
    m = manager(num_pages=2)
    m.admit("a")
    m.extend("a", PAGE_SIZE)
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.extend("b", 2 * PAGE_SIZE)
    assert m.length("b") == 0 and m.groups[0].tables["b"] == []
    assert m.groups[0].pool.n_free == 1
    m.check()


def test_slots_are_exclusive_and_reused():
    m = manager(num_slots=2)
    s1, s2 = m.admit("a"), m.admit("b")
    assert s1 != s2
    with pytest.raises(OutOfSlots):
        m.admit("c")
    with pytest.raises(RuntimeError, match="already live"):
        m.admit("a")
    m.release("a")
    assert m.admit("c") == s1
    m.check()


def test_window_gives_pages_back_once_passed():
    window = 70
    m = manager(num_pages=4, window=window)
    m.admit("r")
    grown = 0
    for length in range(1, 600):
        m.extend("r", length)
        grown = max(grown, m.groups[0].pool.n_used) if False else grown
        table = m.groups[1].tables["r"]
        held = [i for i, p in enumerate(table) if p >= 0]
        # every page that a query at position `length` or later can read is still mapped
        first_key = max(0, length - window + 1)
        assert held and held[0] <= first_key // PAGE_SIZE
        # and nothing older than one page before the window is kept after the next step
        assert len(held) <= (window + PAGE_SIZE - 1) // PAGE_SIZE + 2
        if m.groups[0].pool.n_free == 0 and len(m.groups[0].tables["r"]) * PAGE_SIZE == length:
            break                                # the full-attention group is the one that fills
    assert m.groups[1].pool.high_water <= 4
    m.check()


def test_random_orders_keep_every_invariant():
    rng = random.Random(7)
    for trial in range(30):
        m = manager(num_pages=rng.randint(3, 12), num_slots=rng.randint(1, 5),
                    window=rng.choice([None, 40, 130]))
        live = {}
        counter = 0
        for _ in range(300):
            action = rng.random()
            if action < 0.25 and m.free_slots:
                counter += 1
                name = f"q{counter}"
                m.admit(name)
                live[name] = 0
            elif action < 0.8 and live:
                name = rng.choice(sorted(live))
                target = live[name] + rng.randint(1, 150)
                if m.pages_short(name, target):
                    with pytest.raises(OutOfPages):
                        m.extend(name, target)
                else:
                    m.extend(name, target)
                    live[name] = target
                assert m.length(name) == live[name]
            elif live:
                name = rng.choice(sorted(live))
                m.release(name)
                del live[name]
            m.check()
        for name in list(live):
            m.release(name)
        m.check()
        assert all(g.pool.n_used == 0 for g in m.groups) and m.free_slots == m.num_slots


def test_block_table_rows_as_one_array_follow_the_lists():
    """The array form keeps a request's row between steps: it must notice growth, pages a
    window handed back, and a name that comes back after a release."""
    import numpy as np
    from flyweight_b200.cache.manager import CacheManager
    from flyweight_b200.parts.base import PagedKV
    cache = CacheManager([PagedKV(2, 16, 0), PagedKV(2, 16, 100)], num_pages=12, num_slots=3)
    cache.admit("a"); cache.admit("b")
    cache.extend("a", 70); cache.extend("b", 10)
    for _ in range(3):
        for g in range(2):
            want = np.asarray(cache.block_table(g, ["a", "b"], 5), dtype=np.int32)
            assert np.array_equal(cache.block_table_array(g, ["a", "b"], 5), want)
        cache.extend("a", cache.length("a") + 90)          # grows; the window group lets pages go
        cache.release_passed("a")
    cache.release("a")
    cache.admit("a"); cache.extend("a", 5)                   # the name is back with other pages
    for g in range(2):
        want = np.asarray(cache.block_table(g, ["b", "a"], 3), dtype=np.int32)
        assert np.array_equal(cache.block_table_array(g, ["b", "a"], 3), want)
    cache.check() if hasattr(cache, "check") else None


def test_fixed_states_of_different_dtypes_get_pools_of_their_own_and_are_zeroed_together():
    import torch
    specs = [FixedState((4, 2)), PagedKV(1, 16), FixedState((3,), dtype=torch.bfloat16), FixedState((5,))]
    cache = CacheManager(specs, num_pages=4, num_slots=3, device="cpu")
    states = [cache.layer_caches[i].state for i in (0, 2, 3)]
    assert [s.dtype for s in states] == [torch.float32, torch.bfloat16, torch.float32]
    assert [tuple(s.shape) for s in states] == [(3, 4, 2), (3, 3), (3, 5)]
    for state in states:
        state.fill_(7)
    slot = cache.admit("a")
    for state in states:
        assert float(state[slot].float().abs().sum()) == 0.0            # the slot handed out is clean
        assert all(float(state[other].float().min()) == 7.0 for other in range(3) if other != slot)
    states[0][slot].fill_(1)
    assert float(states[2][slot].sum()) == 0.0 and float(states[1][slot].float().sum()) == 0.0   # no overlap


def test_room_for_one_more_token_counts_the_requests_at_a_page_edge():
    from flyweight_b200.cache import PAGE_SIZE, CacheManager
    from flyweight_b200.parts import PagedKV
    cache = CacheManager([PagedKV(1, 16)], num_pages=5, num_slots=4, device=None)
    for name, length in (("a", PAGE_SIZE), ("b", PAGE_SIZE), ("c", 10)):
        cache.admit(name)
        cache.extend(name, length)
    assert cache.groups[0].pool.n_free == 2
    assert cache.room_for_one_more(["a", "b", "c"], width=4)          # two at an edge, two pages free
    assert not cache.room_for_one_more(["a", "b", "c"], width=1)      # a table of two pages is too wide
    cache.admit("d")
    cache.extend("d", 1)
    assert not cache.room_for_one_more(["a", "b", "c"], width=4)      # one page free, two wanted
    assert cache.room_for_one_more(["a", "c", "d"], width=4)
    assert cache.grow("a", 1) == (cache.slot("a"), PAGE_SIZE) and cache.length("a") == PAGE_SIZE + 1
    assert cache.groups[0].pool.n_free == 0 and not cache.room_for_one_more(["b"], width=4)
    cache.check()


def test_advancing_token_by_token_keeps_the_tables_of_the_general_way():
    """``advance_one`` (the short way of a decode step that follows its predecessor) against
    ``pages_short`` + ``extend`` (what a planned step does): the same tables in a group with a window
    and in one without, pages passed by the window given back at the same token."""
    from flyweight_b200.cache import PAGE_SIZE
    short, general = manager(num_pages=12, window=70), manager(num_pages=12, window=70)
    for m in (short, general):
        for name, length in (("a", 3), ("b", PAGE_SIZE)):
            m.admit(name)
            m.extend(name, length)
    for step in range(5 * PAGE_SIZE):
        assert short.room_for_one_more(["a", "b"], width=8)
        changed = {name: short.advance_one(name) for name in ("a", "b")}
        for name in ("a", "b"):
            before = [list(group.tables[name]) for group in general.groups]
            assert general.pages_short(name, general.length(name) + 1) == 0
            general.extend(name, general.length(name) + 1, checked=True)
            assert changed[name] == (before != [group.tables[name] for group in general.groups])
        for mine, theirs in zip(short.groups, general.groups):
            for name in ("a", "b"):
                assert [p >= 0 for p in mine.tables[name]] == [p >= 0 for p in theirs.tables[name]]
            assert mine.pool.n_used == theirs.pool.n_used
        short.check()
    assert short.groups[1].pool.n_used < short.groups[0].pool.n_used      # the window gave pages back
    assert not short.room_for_one_more(["a", "b"], width=5)              # a table of six pages is too wide
