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


def test_a_state_slot_is_taken_by_the_first_reserve_and_given_back_by_reset_and_release():
    states = StateSlots([None, StateNeed((4,))], max_requests=2)
    m = CacheManager([FULL, None], page_size=4, num_pages=6, state_slots=states)
    assert m.needs_state_slot
    waiting = [m.new_request() for _ in range(50)]            # requests that only wait hold nothing
    assert all(r.state_slot == -1 and not m.holds(r) for r in waiting) and states.num_free == 2
    a, b, c = waiting[:3]
    assert m.reserve(a, 10) and m.reserve(b, 3)
    assert {a.state_slot, b.state_slot} == {0, 1} and m.holds(a)
    # no slot left: nothing fits, nothing is admitted, and a reserve changes nothing
    assert m.room(c, 0) == 0 and not m.admits(1, [0]) and not m.reserve(c, 1)
    assert c.state_slot == -1 and len(c.tables[0]) == 0 and m.num_free(0) == 6 - 3 - 1
    assert m.room(a, 10) == 4 * (3 + 2) - 10                  # a has its slot: pages alone count
    m.reset(a)                                                # preemption: pages and slot go back, the request stays
    assert len(a.tables[0]) == 0 and a.live and a.state_slot == -1 and not m.holds(a) and states.num_free == 1
    assert m.admits(4, [0]) and m.reserve(c, 4) and c.state_slot >= 0
    m.truncate(c, 0)                                          # a step that did not run: pages back, the slot stays
    assert c.state_slot >= 0 and m.holds(c)
    m.release(c)
    assert states.num_free == 1 and m.reserve(a, 2) and a.state_slot >= 0
    with pytest.raises(InvalidArgument, match="released request"):
        m.reserve(c, 1)
    # a model without such state never needs a slot
    plain = CacheManager([FULL], page_size=4, num_pages=6, state_slots=StateSlots([None], max_requests=1))
    rs = [plain.new_request() for _ in range(3)]
    assert not plain.needs_state_slot and all(plain.reserve(r, 4) for r in rs) and all(r.state_slot == -1 for r in rs)


def test_a_window_group_gets_the_pages_it_can_use_and_the_budget_goes_to_the_rest():
    full_bytes, win_bytes = 2 * 2 * 8 * 16 * 4, 2 * 1 * 8 * 32 * 4
    # 4 requests, window 20 and steps of 12 tokens: blocks_for(32, 8) + 2 = 6 pages each
    m = CacheManager([FULL, WIN], page_size=8, budget_bytes=24 * win_bytes + 100 * full_bytes + 7,
                     window_requests=4, window_step_tokens=12)
    assert m.group_pages == [100, 24] and m.num_pages == 100 and m.bytes_per_page == full_bytes
    assert [p.num_blocks for p in m.pools] == [100, 24]
    assert m.max_tokens_per_request() == 800                  # the window group bounds no request's length
    same = CacheManager([FULL, WIN], page_size=8, num_pages=10)
    assert same.group_pages == [10, 10]                       # not asked for: every group alike
    capped = CacheManager([FULL, WIN], page_size=8, num_pages=5, window_requests=4, window_step_tokens=12)
    assert capped.group_pages == [5, 5]                       # never more than the others
    only = CacheManager([WIN], page_size=8, num_pages=50, window_requests=2)
    assert only.group_pages == [2 * (3 + 2)] and only.max_tokens_per_request() == 2 ** 31 - 1
    with pytest.raises(CapacityError, match="beside the window"):
        CacheManager([FULL, WIN], page_size=8, budget_bytes=24 * win_bytes, window_requests=4, window_step_tokens=12)
    # a long request runs through a small window group: its pages come back as the window passes them
    r = m.new_request()
    for at in range(12, 400, 12):
        assert m.reserve(r, at)
        m.advance_window(r, at)
        assert m.group_pages[1] - m.num_free(1) <= 6
    m.release(r)
    assert [p.num_free for p in m.pools] == [100, 24]


@pytest.mark.parametrize("seed", range(25))
def test_no_page_is_lost_held_twice_or_freed_twice_under_random_orders(seed):
    rng = random.Random(seed)
    page = rng.choice([4, 8, 16])
    states = StateSlots([StateNeed((2,)), None, None], max_requests=rng.randint(2, 6))
    m = CacheManager([FULL, WIN, FULL], page_size=page, num_pages=rng.randint(6, 40), state_slots=states,
                     window_requests=rng.choice([None, 2, 6]), window_step_tokens=3 * page)
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
                if r.state_slot < 0:
                    assert not m.holds(r)
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
        # every state slot has one owner or is free; a request that covers tokens has one
        owned = [r.state_slot for r, _ in live.values() if r.state_slot >= 0]
        assert len(owned) == len(set(owned)) and len(owned) + states.num_free == states.max_requests
        assert all(r.state_slot >= 0 for r, n in live.values() if n > 0)
    for r, _ in list(live.values()):
        m.release(r)
    assert all(p.num_free == p.num_blocks for p in m.pools) and states.num_free == states.max_requests


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
