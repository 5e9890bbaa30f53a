"""-m "not gpu": the cache manager -- no page lost, held twice or freed twice, under random orders of requests; groups
with different needs; windows give pages back; state slots."""
import random

import numpy as np
import pytest

from mashbox_b200.cache.manager import CacheManager, CacheNeed, StateNeed
from mashbox_b200.cache.pages import Pool
from mashbox_b200.errors import CacheError


def manager(pages=12, page=4, requests=4, window=10, context=0):
    needs = {0: CacheNeed.keys_and_values(2, 16), 1: CacheNeed.keys_and_values(2, 16, window), 2: CacheNeed.keys_and_values(2, 16), 3: None}
    return CacheManager(needs, {3: StateNeed((5,), "float32")}, page, pages, requests, context)


def test_pool_refuses_double_free_and_reuses_last_freed_first():
    p = Pool(3)
    a, b = p.take(), p.take()
    p.give(a)
    with pytest.raises(CacheError):
        p.give(a)
    with pytest.raises(CacheError):
        p.give(2)
    assert p.take() == a                      # last in, first out: a freed page is used again at once
    p.take()
    with pytest.raises(CacheError):
        p.take()
    p.check()


def test_groups_by_need():
    m = manager()
    assert len(m.groups) == 2
    full = m.groups[m.group_of[0]]
    assert full.cache_ids == [0, 2] and m.group_of[2] == m.group_of[0] and m.group_of[1] != m.group_of[0]
    assert 3 not in m.group_of and m.state_needs[3].shape == (5,)


def test_block_tables_grow_by_pages_and_release_returns_everything():
    m = manager()
    r = m.admit("a")
    m.extend("a", 5)
    m.commit("a", 5)
    full = m.groups[m.group_of[0]]
    assert (full.table[r.row, :2] >= 0).all() and (full.table[r.row, 2:] == -1).all()
    m.extend("a", 3)                                      # 8 tokens: still 2 pages
    m.commit("a", 3)
    assert full.pool.n_free == 10
    m.extend("a", 1)
    assert full.pool.n_free == 9 and m.length("a") == 8   # reserved, not committed
    m.commit("a", 1)
    m.check()
    m.release("a")
    assert m.free_pages() == [12, 12] and m.rows.n_free == 4 and m.state_slots.n_free == 4
    m.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager(pages=12, page=4, window=10)
    r = m.admit("a")
    win = m.groups[m.group_of[1]]
    full = m.groups[m.group_of[0]]
    for _ in range(40):
        m.extend("a", 1)
        m.commit("a", 1)
        m.check()
        n = m.length("a")
        first_needed = max(0, n - 10 + 1) // 4            # the next query (position n) reads keys > n - 10
        held = np.nonzero(win.table[r.row] >= 0)[0]
        assert held.min() == first_needed and held.max() == (n - 1) // 4
        assert win.pool.n_free == 12 - len(held) and len(held) <= 4
        assert full.pool.n_free == 12 - (-(-n // 4))
    m.release("a")
    assert m.free_pages() == [12, 12]


def test_a_long_portion_needs_its_pages_during_the_step_even_with_a_window():
    m = manager(pages=12, page=4, window=6)
    m.admit("a")
    assert m.pages_needed("a", 30) == [8, 8]
    m.extend("a", 30)
    assert m.free_pages() == [4, 4]
    m.commit("a", 30)                                     # after the step only the window's pages stay
    assert sorted(m.free_pages()) == [4, 10]


def test_out_of_pages_is_all_or_nothing():
    m = manager(pages=4, page=4)
    m.admit("a")
    m.admit("b")
    m.extend("a", 9)
    m.commit("a", 9)
    assert not m.can_extend("b", 8)
    before = [g.table.copy() for g in m.groups]
    with pytest.raises(CacheError, match="no free page"):
        m.extend("b", 8)
    assert all((a == g.table).all() for a, g in zip(before, m.groups)) and m.free_pages() == [1, 1]
    m.extend("b", 4)
    m.check()


def test_context_limit_and_unknown_requests():
    m = manager(pages=12, page=4, context=10)
    m.admit("a")
    assert not m.can_extend("a", 11)
    with pytest.raises(CacheError, match="over the context"):
        m.extend("a", 11)
    with pytest.raises(CacheError, match="not live"):
        m.extend("zz", 1)
    with pytest.raises(CacheError, match="already live"):
        m.admit("a")
    for i in range(3):
        m.admit(i)
    assert not m.can_admit()
    with pytest.raises(CacheError):
        m.admit("one too many")
    m.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = manager(pages=rng.choice([6, 9, 16]), page=rng.choice([2, 4, 8]), requests=3, window=rng.choice([3, 7, 12]))
    live, used_pages, counter = {}, set(), 0
    for _ in range(400):
        op = rng.random()
        if op < 0.2 and m.can_admit():
            counter += 1
            m.admit(counter)
            live[counter] = 0
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 9])
            if m.can_extend(rid, n):
                m.extend(rid, n)
                for g in m.groups:
                    used_pages.update(int(x) for x in g.table[m.get(rid).row] if x >= 0)
                if rng.random() < 0.9:
                    m.commit(rid, n)
                    live[rid] += n
                else:                       # a step that took pages and then committed fewer tokens
                    m.commit(rid, 0)
            else:
                with pytest.raises(CacheError):
                    m.extend(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check()
        for rid, n in live.items():
            assert m.length(rid) == n
    for rid in list(live):
        m.release(rid)
    m.check()
    assert all(f == m.num_pages for f in m.free_pages())
    assert len(used_pages) == m.num_pages or len(used_pages) > 0      # pages were handed out again and again
