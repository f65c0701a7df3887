"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; window groups give pages back; slots are handed out once."""

import random

import numpy as np
import pytest

from mini_llm_b200.cache import NO_PAGE, CacheManager, PageError, PagePool, group_entries
from mini_llm_b200.parts.spec import FixedState, PagedKV

FULL = PagedKV(4, 16)
WINDOW = PagedKV(4, 16, window=20)
STATE = FixedState((8,))


def test_pool_all_or_nothing_and_reuse():
    pool = PagePool(4)
    a = pool.alloc(3, "a")
    assert pool.alloc(2, "b") is None and pool.available == 1
    with pytest.raises(PageError):
        pool.free(a, "b")
    pool.free(a, "a")
    with pytest.raises(PageError):
        pool.free([a[0]], "a")
    b = pool.alloc(2, "b")
    assert b[0] == a[-1]              # the page freed last is used again first
    assert pool.reused == 2
    pool.check()


def test_groups_by_need():
    groups = group_entries([FULL, WINDOW, None, FULL, STATE, WINDOW])
    assert [(need, entries) for need, entries in groups] == [(FULL, [0, 3]), (WINDOW, [1, 5]), (STATE, [4])]


def test_block_tables_grow_and_are_given_back():
    m = CacheManager([FULL, FULL], page_size=8, n_pages=6, max_requests=3, max_tokens_per_request=64)
    a, b = m.open(), m.open()
    assert m.reserve(a, 9) and m.pages_held(a) == [2]
    m.commit(a, 9)
    assert m.pages_needed(a, 7) == [0] and m.pages_needed(a, 8) == [1]
    assert m.reserve(b, 32) and m.pages_free() == [0]
    assert not m.reserve(a, 8) and m.pages_held(a) == [2]      # refused: nothing changed
    assert not m.can_reserve(a, 8) and m.can_reserve(a, 7)
    m.check()
    row = m.block_table_row(0, b).copy()
    assert (row[:4] != NO_PAGE).all() and (row[4:] == NO_PAGE).all()
    m.close(b)
    assert m.pages_free() == [4] and (m.block_table_row(0, b) == NO_PAGE).all()
    assert m.reserve(a, 8)
    assert m.block_table_row(0, a)[2] in row[:4]               # a page of b is used again
    with pytest.raises(PageError):
        m.close(b)
    with pytest.raises(PageError):
        m.commit(a, 9)                                         # beyond what was reserved
    m.check()


def test_room_for_gives_the_need_or_none():
    """``room_for`` answers like ``can_reserve`` and hands back what ``pages_needed`` would;
    ``reserve`` given that need does what it does without it; pages set aside count as taken."""
    m = CacheManager([FULL, STATE, WINDOW], page_size=8, n_pages=[4, 0, 3], max_requests=2, max_tokens_per_request=40)
    a = m.open()
    assert m.room_for(a, 9) == m.pages_needed(a, 9) == [2, 0, 2]
    assert m.room_for(a, 25) is None and not m.can_reserve(a, 25)          # the second pool has 3 pages
    assert m.room_for(a, 41) is None                                      # more than a request may hold
    assert m.room_for(a, 9, spare=[2, 0, 1]) == [2, 0, 2] and m.room_for(a, 9, spare=[3, 0, 0]) is None
    need = m.room_for(a, 9)
    assert m.reserve(a, 9, need) and m.pages_held(a) == [2, 0, 2] and m.room_for(a, 0) == [0, 0, 0]
    m.commit(a, 9)
    m.check()


def test_request_cannot_outgrow_its_positions():
    m = CacheManager([FULL], page_size=4, n_pages=100, max_requests=1, max_tokens_per_request=10)
    s = m.open()
    assert m.open() is None
    assert m.reserve(s, 10) and not m.reserve(s, 11)
    m.commit(s, 10)
    assert not m.reserve(s, 1) and not m.can_reserve(s, 1)


def test_window_group_gives_pages_back_as_it_passes_them():
    m = CacheManager([FULL, WINDOW], page_size=8, n_pages=[32, 9], max_requests=2, max_tokens_per_request=200)
    s = m.open()
    length = 0
    for n in [5, 30, 1, 1, 17, 2, 40, 1]:
        assert m.reserve(s, n), (length, n)
        m.commit(s, n)
        length += n
        m.check()
        full, window = m.pages_held(s)
        assert full == -(-length // 8)
        # the next query (position >= length) sees keys > length - 20: earlier pages are gone
        first_needed = max(0, length - 20 + 1) // 8
        row = m.block_table_row(1, s)
        assert (row[:first_needed] == NO_PAGE).all() and (row[first_needed:-(-length // 8)] != NO_PAGE).all()
        assert window == -(-length // 8) - first_needed <= 4
    assert m.freed_by_window > 0
    m.close(s)
    assert m.pages_free() == [32, 9]
    m.check()


def test_fixed_state_needs_no_pages():
    m = CacheManager([STATE, FULL, STATE], page_size=8, n_pages=4, max_requests=2, max_tokens_per_request=64)
    assert [g.paged for g in m.groups] == [False, True]
    assert m.entry_group == {0: (0, 0), 2: (0, 1), 1: (1, 0)}
    s = m.open()
    assert m.pages_needed(s, 20) == [0, 3]
    assert m.reserve(s, 20)
    m.commit(s, 20)
    m.close(s)
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    m = CacheManager([FULL, WINDOW, FULL], page_size=4, n_pages=[40, 24], max_requests=5, max_tokens_per_request=96)
    live = {}
    refused = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and m.free_slots:
            live[m.open()] = 0
        elif action < 0.3 and live:
            slot = rng.choice(list(live))
            m.close(slot)
            del live[slot]
        elif live:
            slot = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13, 30])
            before = (m.pages_free(), m.pages_held(slot))
            if m.reserve(slot, n):
                if rng.random() < 0.8:
                    m.commit(slot, n)
                    live[slot] += n
                elif rng.random() < 0.5:
                    # the step failed after it had reserved: the request holds the pages of
                    # its committed tokens and no more (an earlier reservation goes back too)
                    m.unreserve(slot)
                    assert m.pages_held(slot)[0] == -(-live[slot] // 4) and m.pages_held(slot)[1] <= before[1][1]
            else:
                refused += 1
                assert (m.pages_free(), m.pages_held(slot)) == before
                if live[slot] + n > 96 or rng.random() < 0.5:
                    m.close(slot)
                    del live[slot]
        m.check()
        for slot, length in live.items():
            assert m.length(slot) == length
    for slot in list(live):
        m.close(slot)
    m.check()
    assert m.pages_free() == [40, 24] and m.free_slots == 5
    assert refused > 0 and m.groups[0].pool.reused > 0


def test_unreserve_gives_back_what_a_failed_step_took_and_pages_that_go_back_are_reported():
    m = CacheManager([FULL, WINDOW], page_size=8, n_pages=[6, 6], max_requests=2, max_tokens_per_request=64)
    freed = []
    m.on_free = lambda group, pages: freed.append((group, list(pages)))
    s = m.open()
    assert m.reserve(s, 10)
    m.commit(s, 10)
    held = m.pages_held(s)
    assert m.reserve(s, 30) and m.pages_held(s) == [5, 5]
    m.unreserve(s)
    assert m.pages_held(s) == held == [2, 2] and m.length(s) == 10 and m.pages_free() == [4, 4]
    assert sorted(len(pages) for _, pages in freed) == [3, 3]
    with pytest.raises(PageError):
        m.commit(s, 7)                       # the reservation is gone
    m.unreserve(s)                           # nothing to give back: no change
    assert m.pages_held(s) == [2, 2]
    assert m.reserve(s, 30)
    m.commit(s, 30)                          # the window group gives pages back as it passes them
    assert any(group == 1 for group, _ in freed[2:])
    m.close(s)
    assert sum(len(pages) for _, pages in freed) == 3 + 3 + 5 + 5 and m.pages_free() == [6, 6]
    m.check()
