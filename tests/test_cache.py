"""Page allocator and cache manager (no GPU): nothing lost, held twice or freed twice."""

import random

import pytest
import torch

from simple_inference_b200.cache import CacheManager, OutOfPages, PageAllocator, pages_for
from simple_inference_b200.parts.base import PagedKVSpec, StateSpec


def test_reservation_then_lazy_allocation_lowest_id_first():
    # behaviours of the reference's allocator test (serving/test_paged_kv_cache.py:26-43)
    a = PageAllocator(4)
    a.reserve("r1", 2)
    assert a.free_pages == 4 and a.reserved_pages == 2 and a.available == 2
    assert a.allocate("r1") == 0 and a.allocate("r1") == 1
    with pytest.raises(OutOfPages):
        a.allocate("r1")                      # reservation used up
    assert not a.can_reserve(3) and a.can_reserve(2)
    with pytest.raises(OutOfPages):
        a.reserve("r2", 3)
    a.reserve("r2", 2)
    assert a.allocate("r2") == 2
    a.release("r1")
    assert a.free_pages == 3 and a.allocate("r2") == 0      # lowest id handed out again
    a.check()


def test_double_free_and_foreign_free_are_errors():
    a = PageAllocator(3)
    a.reserve("x", 2)
    p = a.allocate("x")
    a.free_page("x", p)
    with pytest.raises(RuntimeError):
        a.free_page("x", p)
    a.reserve("y", 1)
    q = a.allocate("y")
    with pytest.raises(RuntimeError):
        a.free_page("x", q)
    a.release("x")
    with pytest.raises(KeyError):
        a.release("x")
    a.check()


def _manager(window=None, pages=16, page_size=4, max_requests=3, max_step=8, state=False):
    specs = [PagedKVSpec(2, 16, None), PagedKVSpec(2, 16, None)]
    if window:
        specs.append(PagedKVSpec(2, 16, window))
    if state:
        specs.append(StateSpec((5,), "float32"))
    return CacheManager(specs, page_size, pages, max_requests, max_step, torch.float32, "cpu")


def test_groups_tables_and_slots():
    m = _manager(window=6, state=True)
    assert len(m.groups) == 2                           # all-keys group and windowed group
    assert m.groups[0].entries == [0, 1] and m.groups[1].entries == [2]
    assert m.groups[0].pool.shape == (2, 17, 2, 2, 4, 16)
    views = m.layer_caches()
    assert views[0].group == 0 and views[2].group == 1 and views[3].state.shape == (4, 5)
    m.state[3][1].fill_(7.0)                            # dirt from an earlier tenant of slot 1
    s0 = m.admit("a", 20)
    s1 = m.admit("b", 9)
    assert (s0, s1) == (0, 1)
    assert float(m.state[3][1].abs().sum()) == 0.0      # a slot is zeroed when handed out
    assert m.extend("a", 5) == 0 and m.extend("a", 3) == 5
    assert m.block_table("a", 0) == [0, 1]
    m.extend("b", 1)
    assert m.block_table("b", 0) == [2]
    assert m.write_slot("a", 0, 6) == 1 * 4 + 2
    m.release("a")
    assert m.free_slots == 2
    s2 = m.admit("c", 4)
    assert s2 == 0
    m.extend("c", 4)
    assert m.block_table("c", 0) == [0]                 # a's page is used again
    with pytest.raises(KeyError):
        m.release("a")
    m.check()


def test_window_gives_pages_back_and_reuses_them():
    m = _manager(window=6, pages=8, page_size=4, max_step=4)
    g = m.groups[1]
    assert g.pages_needed(100, 4) == pages_for(6 + 4 - 1, 4) + 1 == 4
    m.admit("a", 100) if m.fits_at_all(100) else None
    # the all-keys group cannot hold 100 tokens in 8 pages
    assert not m.fits_at_all(100)
    m = CacheManager([PagedKVSpec(2, 16, 6)], 4, 8, 2, 4, torch.float32, "cpu")
    m.admit("a", 100)
    seen = set()
    for step in range(25):
        m.extend("a", 4)
        table = m.block_table("a", 0)
        live = [p for p in table if p >= 0]
        assert len(live) <= 4
        start = step * 4
        first_needed = max(0, start - 6 + 1)
        assert all(table[lp] >= 0 for lp in range(first_needed // 4, len(table)))
        seen.update(live)
        m.check()
    assert m.length("a") == 100 and len(seen) <= 5       # a handful of pages, used over and over
    m.release("a")
    assert m.free_pages(0) == 8


def test_out_of_pages_and_slots():
    m = _manager(pages=4, page_size=4, max_requests=2)
    assert m.can_admit(16) and not m.can_admit(17) and not m.fits_at_all(17)
    m.admit("a", 12)
    assert not m.can_admit(8) and m.can_admit(4)
    with pytest.raises(OutOfPages):
        m.admit("b", 8)
    m.admit("b", 4)
    assert not m.can_admit(1)                           # no slot left, and no page either
    m.extend("a", 8)
    with pytest.raises(ValueError):
        m.extend("a", 9)                                # more than max_step_tokens
    m.extend("a", 4)
    with pytest.raises(OutOfPages):
        m.extend("a", 1)                                # beyond its reservation
    m.reserve_to("b", 4)
    with pytest.raises(OutOfPages):
        m.reserve_to("b", 5)                            # nothing left to promise
    m.release("a")
    m.reserve_to("b", 12)
    m.extend("b", 8)
    m.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 5, 12])
    specs = [PagedKVSpec(1, 16, None), PagedKVSpec(1, 16, window)]
    m = CacheManager(specs, rng.choice([2, 4, 8]), 24, 4, 8, torch.float32, "cpu")
    live: dict[int, int] = {}     # request -> tokens it may still take
    next_id = 0
    for _ in range(400):
        action = rng.random()
        if action < 0.3:
            total = rng.randint(1, 40)
            if m.can_admit(total):
                m.admit(next_id, total)
                live[next_id] = total
                next_id += 1
            else:
                with pytest.raises(OutOfPages):
                    m.admit(next_id, total)
        elif action < 0.85 and live:
            r = rng.choice(list(live))
            if live[r] > 0:
                n = rng.randint(1, min(8, live[r]))
                m.extend(r, n)
                live[r] -= n
        elif live:
            r = rng.choice(list(live))
            m.release(r)
            del live[r]
        m.check()
        for g in m.groups:
            owned = [p for req in g.requests for p in g.allocator.owned(req)]
            assert len(owned) == len(set(owned))
            assert len(owned) + g.allocator.free_pages == g.num_pages
    for r in list(live):
        m.release(r)
    m.check()
    assert all(g.allocator.free_pages == g.num_pages for g in m.groups) and m.free_slots == 4


def test_a_spec_of_another_kind_shapes_its_own_pages_and_names_its_own_page_size():
    """The manager only counts pages: a cache kind it has never seen (one vector per token, in
    pages of its own size) says how a page is shaped; groups of different page sizes live side
    by side, each with tables and allocators of its own."""
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class VectorPerToken:
        width: int
        window: int | None = None
        page_size: int | None = 8
        storage = "pages"

        def page_shape(self, page_size):
            return (page_size, self.width)

    specs = [PagedKVSpec(2, 16), VectorPerToken(5), PagedKVSpec(2, 16), VectorPerToken(5), None,
             StateSpec((3,))]
    m = CacheManager(specs, 4, lambda page: 64 // page, 2, 16, torch.float32, "cpu")
    assert [g.entries for g in m.groups] == [[0, 2], [1, 3]]
    assert [g.page_size for g in m.groups] == [4, 8] and [g.num_pages for g in m.groups] == [16, 8]
    assert m.groups[0].pool.shape == (2, 17, 2, 2, 4, 16) and m.groups[1].pool.shape == (2, 9, 8, 5)
    views = m.layer_caches()
    assert views[1].pool.shape == (9, 8, 5) and views[1].page_size == 8 and views[1].group == 1
    assert views[4] is None and views[5].state.shape == (3, 3)
    m.admit("a", 30)
    m.extend("a", 13)
    assert len(m.block_table("a", 0)) == 4 and len(m.block_table("a", 1)) == 2
    assert m.write_slot("a", 1, 12) == m.block_table("a", 1)[1] * 8 + 4
    assert not m.can_admit(40) and m.can_admit(32)      # 8 pages of 4 and 4 pages of 8 are promised
    m.check()
    m.release("a")
    assert m.free_pages(0) == 16 and m.free_pages(1) == 8
    with pytest.raises(ValueError):
        @dataclass(frozen=True)
        class Odd:
            storage = "elsewhere"
        CacheManager([Odd()], 4, 8, 1, 4, torch.float32, "cpu")
