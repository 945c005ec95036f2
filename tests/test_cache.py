"""The cache manager on the host: pages, tables, windows, state slots, invariants."""

import random

import pytest
import torch

from socrates_b200.cache import (CacheManager, CacheNeeds, OutOfPages, PageAllocator, PagedKVSpec,
                                 StateSpec, pages_for)


def test_pages_for():
    assert [pages_for(n, 16) for n in (0, 1, 15, 16, 17, 32, 33)] == [0, 1, 1, 1, 2, 2, 3]


def test_allocator_round_trip_and_errors():
    a = PageAllocator(4)
    got = a.alloc(3)
    assert got == [1, 2, 3] and 0 not in got and a.n_free == 1
    with pytest.raises(OutOfPages):
        a.alloc(2)
    assert a.n_free == 1                                   # a failed alloc changes nothing
    a.free([2])
    assert a.alloc(1) == [2]                               # last freed, first reused
    with pytest.raises(ValueError):
        a.free([0])
    with pytest.raises(ValueError):
        a.free([4])                                        # never allocated
    with pytest.raises(ValueError):
        a.free([1, 1])
    assert a.n_used == 3                                   # a failed free changes nothing
    a.free([1, 2, 3])
    with pytest.raises(ValueError):
        a.free([1])                                        # freed twice
    a.check()


def manager(num_pages=12, max_rows=4, max_len=128, window=None, state=False):
    needs = [CacheNeeds(PagedKVSpec(2, 16, None)),
             CacheNeeds(PagedKVSpec(2, 16, window), StateSpec((3,)) if state else None),
             CacheNeeds(PagedKVSpec(2, 16, None))]
    return CacheManager(needs, max_rows, max_len, 16, num_pages, torch.float32, "cpu")


def test_groups_by_need():
    m = manager(window=None)
    assert len(m.groups) == 1 and m.groups[0].entries == [0, 1, 2]
    assert m.pools(1)[0].shape == (13, 2, 16, 16)
    m = manager(window=20)
    assert len(m.groups) == 2
    assert m.groups[m.group_of_entry[0]].entries == [0, 2]
    assert m.groups[m.group_of_entry[1]].entries == [1]
    assert m.window(1) == 20 and m.window(0) is None


def test_lazy_reserve_is_all_or_nothing():
    m = manager(num_pages=3, window=20)
    m.assign(0)
    assert m.reserve(0, 40)                                # 3 pages in each group
    assert m.free_pages() == [0, 0]
    m.assign(1)
    assert not m.reserve(1, 1)
    assert m.free_pages() == [0, 0] and m.groups[0].owned(1) == []
    m.check()
    with pytest.raises(ValueError):
        m.reserve(0, 129)                                  # beyond the row's table


def test_window_gives_pages_back():
    m = manager(num_pages=8, window=20)
    full, win = m.groups[m.group_of_entry[0]], m.groups[m.group_of_entry[1]]
    m.assign(0)
    assert m.reserve(0, 48)
    m.commit(0, 48)
    # next query is at 48 and sees keys 29..48: block 0 (slots 0..15) is gone, block 1 stays
    assert win.row_pages[0][0] == 0 and win.row_pages[0][1] != 0
    assert len(win.owned(0)) == 2 and len(full.owned(0)) == 3
    assert int(win.host_table[0, 0]) == 0
    # growing further only asks the windowed group for blocks it can still see
    assert m.pages_needed(0, 49) == [1, 1]
    m.commit(0, 48)
    assert m.reserve(0, 100)
    m.commit(0, 100)
    assert len(win.owned(0)) == 2 and len(full.owned(0)) == 7
    m.check()
    m.release(0)
    assert m.free_pages() == [8, 8]
    m.check()


def test_tables_follow_ownership_and_move_row():
    m = manager(state=True, window=None)
    m.assign(0)
    m.assign(2)
    m.reserve(0, 20)
    m.reserve(2, 5)
    m.commit(0, 20)
    m.commit(2, 5)
    m.state(1)[2] = torch.tensor([1.0, 2.0, 3.0])
    pages = list(m.groups[0].row_pages[2])
    k_ptr = m.pools(0)[0].data_ptr()
    m.flush()
    assert m.groups[0].table[2, 0] == pages[0]
    m.move_row(2, 1)
    m.flush()
    assert m.groups[0].row_pages[1] == pages and m.groups[0].row_pages[2] == []
    assert m.lengths[1] == 5 and m.lengths[2] == 0 and m.active[1] and not m.active[2]
    assert int(m.groups[0].table[1, 0]) == pages[0] and int(m.groups[0].table[2, 0]) == 0
    assert m.state(1)[1].tolist() == [1.0, 2.0, 3.0]
    assert m.pools(0)[0].data_ptr() == k_ptr               # the pages themselves never move
    with pytest.raises(ValueError):
        m.move_row(1, 0)                                   # destination in use
    m.check()


def test_state_slot_is_zeroed_on_assign():
    m = manager(state=True)
    m.assign(3)
    m.state(1)[3] = 7.0
    m.release(3)
    m.assign(3)
    assert m.state(1)[3].abs().sum() == 0


def test_row_errors():
    m = manager()
    with pytest.raises(ValueError):
        m.reserve(0, 4)                                    # not assigned
    m.assign(0)
    with pytest.raises(ValueError):
        m.assign(0)
    m.reserve(0, 10)
    m.commit(0, 10)
    with pytest.raises(ValueError):
        m.commit(0, 5)
    m.release(0)
    with pytest.raises(ValueError):
        m.release(0)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    """Requests come, grow by random portions, move and go in random order; after every
    operation no page is lost, held twice or freed twice, and tables match ownership."""
    rng = random.Random(seed)
    window = rng.choice([None, 20, 37])
    m = manager(num_pages=rng.choice([6, 10, 24]), max_rows=5, max_len=160, window=window)
    live = {}
    for _ in range(400):
        op = rng.random()
        free_rows = [r for r in range(5) if not m.active[r]]
        if op < 0.25 and free_rows:
            r = rng.choice(free_rows)
            m.assign(r)
            live[r] = 0
        elif op < 0.75 and live:
            r = rng.choice(list(live))
            new_len = min(160, live[r] + rng.choice([1, 1, 1, 2, 7, 16, 33]))
            before = m.free_pages()
            if m.reserve(r, new_len):
                m.commit(r, new_len)
                live[r] = new_len
            else:
                assert m.free_pages() == before
        elif op < 0.9 and live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        elif live and free_rows:
            src, dst = rng.choice(list(live)), rng.choice(free_rows)
            m.move_row(src, dst)
            live[dst] = live.pop(src)
        m.check()
        for r, n in live.items():
            assert m.lengths[r] == n
            for g in m.groups:                              # every slot a later query can see has a page
                for b in range(g.first_needed_block(n), pages_for(n, 16)):
                    assert g.row_pages[r][b] != 0
    for r in list(live):
        m.release(r)
    m.check()
    assert all(f == g.allocator.num_pages for f, g in zip(m.free_pages(), m.groups))
