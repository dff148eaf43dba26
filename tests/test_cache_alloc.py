"""Cache bookkeeping on the host: no slot or page is lost, held twice or freed twice."""
import random

import pytest

from llm_infer_engine_b200.cache.allocator import CacheError, FreeList, PageTableHost


def test_free_list_basics():
    fl = FreeList(4, "slot")
    got = [fl.take() for _ in range(4)]
    assert got == [0, 1, 2, 3] and fl.n_free == 0
    with pytest.raises(CacheError, match="no free slot"):
        fl.take()
    fl.give_back(2)
    with pytest.raises(CacheError, match="freed twice"):
        fl.give_back(2)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back(9)
    fl.give_back(0)
    assert fl.take() == 0 and fl.take() == 2          # given back, handed out again, lowest first
    fl.check()
    with pytest.raises(CacheError, match="wanted"):
        FreeList(2, "page").take_many(3)


def test_random_workload_keeps_the_books_straight():
    rng = random.Random(0)
    page = 64
    table = PageTableHost(n_pages=40, page_size=page, max_pages_per_seq=12)
    slots = FreeList(6, "slot")
    live = {}
    for step in range(3000):
        action = rng.random()
        if action < 0.25 and slots.n_free:
            s = slots.take()
            table.open_slot(s)
            live[s] = 0
        elif action < 0.80 and live:
            s = rng.choice(list(live))
            new_len = min(live[s] + rng.choice([1, 1, 1, 5, 70, 200]), 12 * page)
            need = table.pages_needed(s, live[s], new_len)
            if need <= table.pages.n_free:
                mapped = table.grow(s, live[s], new_len)
                assert len(mapped) == need
                live[s] = new_len
                held = table.held_pages(s)
                assert sorted(held) == list(range((new_len + page - 1) // page))      # every position is mapped
            else:
                with pytest.raises(CacheError):
                    table.grow(s, live[s], new_len)
        elif live:
            s = rng.choice(list(live))
            table.close_slot(s)
            slots.give_back(s)
            del live[s]
        table.check()
        slots.check()
        assert table.pages.n_held == sum((l + page - 1) // page for l in live.values())
    for s in list(live):
        table.close_slot(s)
        slots.give_back(s)
    assert table.pages.n_free == 40 and slots.n_free == 6
    with pytest.raises(CacheError, match="not open"):
        table.close_slot(0)
    table.open_slot(0)
    with pytest.raises(CacheError, match="opened twice"):
        table.open_slot(0)
    with pytest.raises(CacheError, match="per-sequence limit"):
        table.grow(0, 0, 12 * page + 1)


def test_window_group_gives_pages_back():
    page, window = 64, 100
    table = PageTableHost(n_pages=8, page_size=page, max_pages_per_seq=100, window=window)
    table.open_slot(0)
    length = 0
    table.grow(0, 0, 300)                       # a long prompt needs all its pages during the step
    length = 300
    assert table.pages.n_held == 5
    table.trim(0, length)                       # the next token reads positions 201..300
    assert sorted(table.held_pages(0)) == [3, 4]
    for _ in range(2000):                       # far more tokens than 8 pages could hold without trimming
        table.grow(0, length, length + 1)
        length += 1
        table.trim(0, length)
        first_needed = max(0, length + 1 - window) // page
        assert min(table.held_pages(0)) == first_needed
        assert table.pages.n_held <= (window + page - 1) // page + 1
        table.check()
    table.close_slot(0)
    assert table.pages.n_free == 8
