"""Cache manager: no page lost, held twice or freed twice; windows give pages
back; groups with different needs have pools of their own; state slots."""

import random

import pytest

from freetoken_b200.cache import (CacheManager, NoFreeSlot, OutOfPages, PageAccountingError,
                                  PagedKVNeed, PagePool, StateNeed)


def test_pool_hands_out_every_page_once_and_reuses_freed_ones_first():
    pool = PagePool(5)
    a = pool.allocate(3, "a")
    assert a == [1, 2, 3] and pool.free_pages == 2
    pool.release([2], "a")
    assert pool.allocate(1, "b") == [2]                  # a freed page is the next one handed out
    with pytest.raises(OutOfPages):
        pool.allocate(3, "c")
    with pytest.raises(PageAccountingError, match="held by"):
        pool.release([1], "b")                            # a stranger frees it
    pool.release([1, 3], "a")
    with pytest.raises(PageAccountingError, match="nobody holds"):
        pool.release([1], "a")                            # freed twice
    pool.check()


def full(nkv=2, d=16):
    return PagedKVNeed(nkv, d, None)


def test_grow_advance_release_accounting():
    m = CacheManager([full(), full()], page_size=4, num_pages=6, max_slots=2, max_seq_len=24)
    assert len(m.paged_groups) == 1 and m.paged_groups[0].stops == [0, 1]   # equal needs share pages
    m.admit("a")
    m.grow("a", 9)                                        # 3 pages
    assert m.held_pages("a") == [3] and m.free_pages() == [3]
    m.advance("a", 9)
    m.grow("a", 10)                                       # still inside page 3
    assert m.held_pages("a") == [3]
    m.advance("a", 1)
    with pytest.raises(PageAccountingError, match="without pages"):
        m.advance("a", 5)
    m.admit("b")
    assert not m.can_grow("b", 13)
    with pytest.raises(OutOfPages):
        m.grow("b", 13)                                   # needs 4, 3 free: nothing is taken
    assert m.held_pages("b") == [0] and m.free_pages() == [3]
    with pytest.raises(NoFreeSlot):
        m.admit("c")
    m.release("a")
    m.grow("b", 13)
    first_row = m.paged_groups[0].block_table[m.slot("b")]
    assert set(first_row[:4].tolist()) & {1, 2, 3}        # a's pages are used again
    m.check_integrity()
    m.release("b")
    assert m.free_pages() == m.total_pages() and m.free_slots == 2
    m.check_integrity()


def test_window_group_gives_pages_back_while_the_request_runs():
    needs = [PagedKVNeed(2, 16, None), PagedKVNeed(2, 16, 6)]      # all keys / the last 6
    m = CacheManager(needs, page_size=4, num_pages=[8, 4], max_slots=1, max_seq_len=32)
    assert len(m.paged_groups) == 2
    m.admit("r")
    for step_tokens in (5, 3, 1, 1, 1, 1, 1, 7):
        new_len = m.length("r") + step_tokens
        m.grow("r", new_len)
        m.advance("r", step_tokens)
        m.check_integrity()
        dead_below = max(0, new_len - 6 + 1) // 4
        assert m.held_pages("r") == [-(-new_len // 4), -(-new_len // 4) - dead_below]
    assert m.length("r") == 20 and m.held_pages("r") == [5, 2]
    assert (m.paged_groups[1].block_table[0, :3] == 0).all()        # passed pages point at the sink
    m.release("r")
    assert m.free_pages() == [8, 4]
    assert m.worst_case_pages(32, 7) == [8, 5]


def test_state_groups_and_fresh_slots():
    needs = [StateNeed((4, 3)), full(), StateNeed((4, 3)), StateNeed((2,), "int32"), None]
    m = CacheManager(needs, page_size=8, num_pages=4, max_slots=3, max_seq_len=32)
    assert [g.stops for g in m.state_groups] == [[0, 2], [3]]
    assert m.state_index[2] == (0, 1) and m.paged_index[1] == (0, 0) and 4 not in m.paged_index
    s1, s2 = m.admit("x"), m.admit("y")
    assert sorted(m.take_fresh_slots()) == sorted([s1, s2]) and m.take_fresh_slots() == []
    m.release("x")
    s3 = m.admit("z")
    assert s3 == s1 and m.take_fresh_slots() == [s3]       # a reused slot must be cleared again


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_double_hold_a_page(seed):
    rng = random.Random(seed)
    needs = [full(), PagedKVNeed(1, 8, rng.choice([5, 9, 16])), full()]
    page = rng.choice([2, 4, 8])
    m = CacheManager(needs, page_size=page, num_pages=[rng.randint(6, 14), rng.randint(6, 14)],
                     max_slots=4, max_seq_len=64)
    live, counter = {}, 0
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            counter += 1
            rid = f"r{counter}"
            m.admit(rid)
            live[rid] = 0
        elif action < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 11])
            new_len = live[rid] + n
            if new_len <= 64 and m.can_grow(rid, new_len):
                m.grow(rid, new_len)
                m.advance(rid, n)
                live[rid] = new_len
            else:
                before = m.free_pages()
                if new_len <= 64:
                    with pytest.raises(OutOfPages):
                        m.grow(rid, new_len)
                    assert m.free_pages() == before       # a refused grow takes nothing
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_integrity()
        for rid, length in live.items():
            assert m.length(rid) == length
    for rid in list(live):
        m.release(rid)
    m.check_integrity()
    assert m.free_pages() == m.total_pages()
