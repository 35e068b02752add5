"""The cache manager on the host: pools, block tables, groups, windows, state slots (CPU)."""
import random

import numpy as np
import pytest

from tiny_inference_engine_b200.cache import FREED, BlockPool, CacheManager, StateSlots, blocks_for
from tiny_inference_engine_b200.errors import CapacityError, InvalidArgument
from tiny_inference_engine_b200.parts import CacheNeed, StateNeed

FULL = CacheNeed("full", 2, 16)
WIN = CacheNeed("window", 1, 32, window=20)


def test_pool_lowest_first_reuse_and_misuse():
    p = BlockPool(4)
    assert [p.allocate() for _ in range(3)] == [0, 1, 2] and p.num_free == 1
    p.release(1)
    assert p.allocate() == 1                       # the page just given back is used again
    p.retain(2)
    p.release(2)
    assert p.ref_count(2) == 1 and p.num_free == 1
    p.release(2)
    assert p.num_free == 2
    with pytest.raises(InvalidArgument, match="already free"):
        p.release(2)
    with pytest.raises(InvalidArgument, match="retain free"):
        p.retain(2)
    with pytest.raises(InvalidArgument, match="outside"):
        p.release(9)
    p.allocate(), p.allocate()
    with pytest.raises(CapacityError, match="full"):
        p.allocate()
    with pytest.raises(InvalidArgument):
        BlockPool(0)


def test_groups_by_need_and_page_bytes():
    m = CacheManager([FULL, None, FULL, WIN, None], page_size=8, num_pages=10)
    assert len(m.groups) == 2
    assert m.groups[0].entries == (0, 2) and m.groups[1].entries == (3,) and m.groups[1].window == 20
    assert m.group_of(2) == 0 and m.group_of(3) == 1 and not m.has_cache(1)
    # float32 bookkeeping without storage: 2 (K,V) * planes * heads * page * dim * 4 bytes
    assert m.bytes_per_page == 2 * 2 * 2 * 8 * 16 * 4 + 2 * 1 * 1 * 8 * 32 * 4
    by_budget = CacheManager([FULL], page_size=16, budget_bytes=10 * 2 * 2 * 16 * 16 * 4 + 5)
    assert by_budget.num_pages == 10
    with pytest.raises(CapacityError, match="smaller than one"):
        CacheManager([FULL], page_size=16, budget_bytes=100)


def test_reserve_is_all_or_nothing_over_groups():
    m = CacheManager([FULL, WIN], page_size=4, num_pages=5)
    a, b = m.new_request(), m.new_request()
    assert m.reserve(a, 9) and [len(t) for t in a.tables] == [3, 3]
    assert m.reserve(a, 5) and [len(t) for t in a.tables] == [3, 3]          # already covered
    assert not m.reserve(b, 12) and [len(t) for t in b.tables] == [0, 0]     # needs 3, only 2 free: nothing changes
    assert m.num_free(0) == 2 and m.num_free(1) == 2
    assert m.reserve(b, 8)
    assert m.room(a, 9) == 3 and m.room(b, 0) == 8
    slots = m.slots(a, 0, 3, 9)
    ids = a.tables[0].view()
    assert list(slots) == [ids[0] * 4 + 3, ids[1] * 4, ids[1] * 4 + 1, ids[1] * 4 + 2, ids[1] * 4 + 3, ids[2] * 4]
    with pytest.raises(InvalidArgument, match="cannot hold"):
        m.slots(a, 0, 0, 13)
    m.truncate(a, 4)
    assert [len(t) for t in a.tables] == [1, 1] and m.num_free(0) == 2
    m.release(a), m.release(b)
    assert m.num_free(0) == 5 and m.num_free(1) == 5
    with pytest.raises(InvalidArgument, match="twice"):
        m.release(a)


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([FULL, WIN], page_size=8, num_pages=12)
    r = m.new_request()
    assert m.reserve(r, 64)
    m.advance_window(r, 64)     # next query at 64 reads keys > 64 - 20 = 44, i.e. from 45: pages 0..4 are done
    full, win = r.tables
    assert full.released == 0 and win.released == 5
    assert list(win.view()[:5]) == [FREED] * 5 and (win.view()[5:] >= 0).all()
    assert m.num_free(0) == 4 and m.num_free(1) == 9
    assert m.room(r, 64) == 32                   # positional: 8 + 4 pages of the full group
    with pytest.raises(InvalidArgument, match="below the window"):
        m.slots(r, 1, 30, 64)
    assert len(m.slots(r, 1, 45, 64)) == 19
    m.truncate(r, 10)                            # never below what the window already gave back
    assert len(full) == 2 and len(win) == 5
    m.release(r)
    assert m.num_free(0) == 12 and m.num_free(1) == 12


def test_reset_keeps_the_request_and_zeroes_its_place():
    states = StateSlots([None, StateNeed((4,))], max_requests=2)
    m = CacheManager([FULL, None], page_size=4, num_pages=6, state_slots=states)
    a, b = m.new_request(), m.new_request()
    assert {a.state_slot, b.state_slot} == {0, 1}
    with pytest.raises(CapacityError, match="state slots"):
        m.new_request()
    m.reserve(a, 10)
    m.reset(a)
    assert len(a.tables[0]) == 0 and a.live and a.state_slot >= 0 and m.num_free(0) == 6
    m.release(a)
    assert states.num_free == 1
    c = m.new_request()
    assert c.state_slot == a.state_slot if a.state_slot >= 0 else True


@pytest.mark.parametrize("seed", range(25))
def test_no_page_is_lost_held_twice_or_freed_twice_under_random_orders(seed):
    rng = random.Random(seed)
    page = rng.choice([4, 8, 16])
    m = CacheManager([FULL, WIN, FULL], page_size=page, num_pages=rng.randint(6, 40))
    live = {}   # request -> tokens covered
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            r = m.new_request()
            live[id(r)] = [r, 0]
        elif op < 0.7 and live:
            r, n = rng.choice(list(live.values()))
            want = n + rng.randint(1, 3 * page)
            before = [len(t) for t in r.tables]
            if m.reserve(r, want):
                live[id(r)][1] = want
                m.advance_window(r, want)
            else:
                assert [len(t) for t in r.tables] == before
        elif op < 0.8 and live:
            r, n = rng.choice(list(live.values()))
            cut = rng.randint(0, n)
            m.truncate(r, cut)
            live[id(r)][1] = min(n, cut)
        elif op < 0.9 and live:
            r, n = rng.choice(list(live.values()))
            m.reset(r)
            live[id(r)][1] = 0
        elif live:
            r, _ = live.pop(rng.choice(list(live)))
            m.release(r)
        # every page has exactly one owner or is free
        for g, pool in enumerate(m.pools):
            held = [b for r, _ in live.values() for b in r.tables[g].held()]
            assert len(held) == len(set(held)), "a page is held twice"
            assert len(held) + pool.num_free == pool.num_blocks, "a page is lost"
            assert all(pool.ref_count(b) == 1 for b in held)
            free = set(range(pool.num_blocks)) - set(held)
            assert all(pool.ref_count(b) == 0 for b in free)
        for r, n in live.values():
            assert len(r.tables[0]) >= blocks_for(n, page)
    for r, _ in list(live.values()):
        m.release(r)
    assert all(p.num_free == p.num_blocks for p in m.pools)


def test_state_slots_misuse():
    s = StateSlots([None], 2)
    a = s.allocate()
    s.release(a)
    with pytest.raises(InvalidArgument, match="while free"):
        s.release(a)
    assert s.bytes_per_slot == 0 and s.tensor(0) is None


def test_workspace_keeps_outgrown_buffers_and_sizes_by_capacity():
    """A flat buffer that has to grow leaves the old one alive (a captured graph may still use its address);
    with a capacity given it never has to."""
    import torch

    from tiny_inference_engine_b200.engine.workspace import Workspace
    ws = Workspace(8, "cpu")
    a = ws.flat("x", 10, torch.float32)
    assert ws.flat("x", 5, torch.float32) is a
    b = ws.flat("x", 50, torch.float32)
    assert b is not a and b.numel() >= 50 and any(t is a for t in ws._retired)
    c = ws.flat("y", 10, torch.float32, capacity=1000)
    assert c.numel() == 1000 and ws.flat("y", 1000, torch.float32, capacity=1000) is c
    z = ws.zeros("z", 4, torch.int32)
    assert not z.any() and ws.zeros("z", 4, torch.int32) is z
    assert ws.rows("r", 8, 3, torch.float32).shape == (8, 3)
    with pytest.raises(ValueError, match="rows asked"):
        ws.rows("r", 9, 3, torch.float32)
