"""Cache manager: no page lost, held twice or freed twice, under random orders of requests;
windows give pages back; state slots."""
import random

import pytest

from allpaca_b200.cache import CacheError, CacheManager, FREED, GroupLayout, OutOfPages, PagePool


def test_pool_is_lifo_and_detects_double_free():
    pool = PagePool(4)
    a, b = pool.alloc(), pool.alloc()
    assert (a, b) == (0, 1) and pool.num_free == 2
    pool.free(a)
    assert pool.alloc() == a            # a page just given back is used again at once
    pool.free(b)
    with pytest.raises(CacheError, match="freed twice"):
        pool.free(b)
    with pytest.raises(CacheError, match="outside"):
        pool.free(9)
    pool.alloc(), pool.alloc(), pool.alloc()
    with pytest.raises(OutOfPages):
        pool.alloc()


def test_append_allocates_by_page_and_slots_follow_the_table():
    m = CacheManager([GroupLayout(page_size=4, num_pages=8)], max_seqs=2)
    m.begin("a")
    assert m.append("a", 5) == 0
    assert len(m.block_table("a", 0)) == 2
    assert m.append("a", 3) == 5 and len(m.block_table("a", 0)) == 2
    assert m.append("a", 1) == 8 and len(m.block_table("a", 0)) == 3
    t = m.block_table("a", 0)
    assert m.slots("a", 0, 3, 3) == [t[0] * 4 + 3, t[1] * 4 + 0, t[1] * 4 + 1]
    assert m.slot("a", 0, 8) == t[2] * 4
    m.check()
    m.free("a")
    assert m.num_free_pages() == 8
    with pytest.raises(CacheError):
        m.free("a")


def test_out_of_pages_changes_nothing():
    m = CacheManager([GroupLayout(4, 3), GroupLayout(4, 2)], max_seqs=2)
    m.begin("a")
    m.append("a", 8)                      # 2 pages in each group; group 1 is now full
    assert not m.can_append("a", 1)
    with pytest.raises(OutOfPages):
        m.append("a", 1)
    assert m.num_tokens("a") == 8 and m.num_free_pages(0) == 1 and m.num_free_pages(1) == 0
    m.check()
    assert m.can_append(None, 4, reserve=[0, 0]) is False
    m.free("a")
    assert m.can_append(None, 8) and not m.can_append(None, 9)
    assert m.can_append(None, 8, reserve=[0, 1]) is False


def test_state_slots_are_limited_and_reused():
    m = CacheManager([GroupLayout(4, 8)], max_seqs=2)
    s0, s1 = m.begin("a"), m.begin("b")
    assert {s0, s1} == {0, 1} and not m.can_begin()
    with pytest.raises(OutOfPages):
        m.begin("c")
    with pytest.raises(CacheError):
        m.begin("a")
    m.free("a")
    assert m.begin("c") == s0
    m.check()


def test_window_pages_are_given_back_once_passed():
    m = CacheManager([GroupLayout(4, 100), GroupLayout(4, 6, window=6)], max_seqs=1)
    m.begin("a")
    m.append("a", 9)                       # pages 0..2 in both groups
    assert m.release_passed("a") == 1      # next row at 9 sees keys 4..9: page 0 is dead
    assert m.block_table("a", 1)[0] == FREED and m.block_table("a", 0)[0] != FREED
    m.check()
    with pytest.raises(CacheError, match="given back"):
        m.slots("a", 1, 2, 1)
    for _ in range(40):                    # a long decode lives on 6 pages of the window group
        m.append("a", 1)
        m.release_passed("a")
        m.check()
    live = [p for p in m.block_table("a", 1) if p != FREED]
    assert len(live) <= 3 and m.num_tokens("a") == 49
    m.free("a")
    assert m.num_free_pages(1) == 6 and m.num_free_pages(0) == 100


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    m = CacheManager([GroupLayout(4, 24), GroupLayout(4, 16, window=10)], max_seqs=5)
    live, next_id = [], 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.can_begin():
            m.begin(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.85 and live:
            r = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 5, 9])
            if m.can_append(r, n):
                m.append(r, n)
                m.release_passed(r)
            else:
                with pytest.raises(OutOfPages):
                    m.append(r, n)
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.free(r)
        m.check()
    for r in live:
        m.free(r)
    m.check()
    assert m.num_free_pages(0) == 24 and m.num_free_pages(1) == 16
