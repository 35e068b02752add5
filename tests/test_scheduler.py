"""The scheduler's decisions, without a model: the test plays the engine's part (CPU).

Cases follow the reference's scheduler tests in spirit (tests/engine/test_batch_scheduler.cpp:88-356
and the randomized simulation tests/engine/test_batch_scheduler_sim.cpp:23-128).
"""
import random

import pytest

from tiny_inference_engine_b200.cache import CacheManager, StateSlots, blocks_for
from tiny_inference_engine_b200.engine import Scheduler, SchedulerConfig, ServingConfig
from tiny_inference_engine_b200.engine.sequence import SeqState, Sequence
from tiny_inference_engine_b200.errors import InvalidArgument
from tiny_inference_engine_b200.parts import CacheNeed, StateNeed
from tiny_inference_engine_b200.sampling import SamplingParams

PAGE = 4


class Rig:
    """Scheduler + cache, and the engine's bookkeeping around them."""

    def __init__(self, pages=64, tokens=16, seqs=4, policy="fcfs", aging=16, watermark=-1, needs=None, slots=None,
                 window_requests=None):
        needs = needs or [CacheNeed("full", 1, 8)]
        self.states = StateSlots([StateNeed((2,))] + [None] * (len(needs) - 1), slots) if slots else None
        self.cache = CacheManager(needs, page_size=PAGE, num_pages=pages, state_slots=self.states,
                                  window_requests=window_requests, window_step_tokens=tokens)
        self.s = Scheduler(self.cache, SchedulerConfig(ServingConfig(tokens, seqs), policy, aging, watermark))
        self.seqs, self.next = [], 0

    def add(self, prompt, max_tokens=4):
        q = Sequence(self.next, list(range(prompt)), prompt, SamplingParams(max_tokens=max_tokens), self.cache.new_request())
        self.next += 1
        self.s.add(q)
        self.seqs.append(q)
        return q

    def step(self):
        b = self.s.schedule()
        self.finish_step(b)
        return [(q.id, n) for q, n in b.seqs]

    def finish_step(self, b):
        for q, n in b.seqs:
            q.num_computed += n
            self.cache.advance_window(q.cache, q.num_computed)
        self.s.complete(b)
        for q, n in b.seqs:
            if q.num_computed == len(q.tokens):
                q.tokens.append(0)
                q.state = SeqState.DECODING
                if q.num_generated >= q.params.max_tokens:
                    self.finish(q)

    def finish(self, q):
        q.state = SeqState.FINISHED
        self.cache.release(q.cache)
        self.s.finish(q)


def test_config_is_checked():
    for bad in (ServingConfig(0, 1), ServingConfig(8, 0), ServingConfig(4, 8)):
        with pytest.raises(InvalidArgument):
            bad.validate()
    c = CacheManager([CacheNeed("full", 1, 8)], page_size=4, num_pages=10)
    with pytest.raises(InvalidArgument, match="policy"):
        Scheduler(c, SchedulerConfig(policy="lifo"))
    with pytest.raises(InvalidArgument, match="aging"):
        Scheduler(c, SchedulerConfig(aging=-1))
    with pytest.raises(InvalidArgument, match="watermark"):
        Scheduler(c, SchedulerConfig(watermark_pages=10))
    assert Scheduler(c, SchedulerConfig()).watermark == 1
    assert Scheduler(CacheManager([CacheNeed("full", 1, 8)], 4, num_pages=1000), SchedulerConfig()).watermark == 10


def test_prompt_is_cut_under_the_token_budget_then_decodes():
    r = Rig(tokens=8)
    a = r.add(19, max_tokens=2)
    assert r.step() == [(0, 8)] and a.state == SeqState.PREFILLING
    assert r.step() == [(0, 8)]
    assert r.step() == [(0, 3)] and a.state == SeqState.DECODING and a.num_generated == 1
    assert r.step() == [(0, 1)] and a.state == SeqState.FINISHED
    assert r.cache.num_free() == 64 and not r.s.has_work()


def test_decodes_come_first_then_prompts_in_progress_then_admission():
    r = Rig(tokens=10, seqs=4)
    a = r.add(3, 8)
    assert r.step() == [(0, 3)]
    b = r.add(14, 8)
    assert r.step() == [(0, 1), (1, 9)]            # a decodes, b takes what is left of the budget
    c = r.add(2, 8)
    assert r.step() == [(0, 1), (1, 5), (2, 2)]    # decode, b's rest, then c is admitted
    assert r.step() == [(0, 1), (1, 1), (2, 1)]


def test_max_seqs_limits_running_requests():
    r = Rig(tokens=16, seqs=2)
    for _ in range(3):
        r.add(2, 3)
    assert r.step() == [(0, 2), (1, 2)]
    assert r.step() == [(0, 1), (1, 1)]
    assert r.step() == [(0, 1), (1, 1)]            # both finish here (3 tokens each)
    assert r.step() == [(2, 2)]


def test_admission_respects_the_watermark_and_stops_at_the_first_that_does_not_fit():
    r = Rig(pages=6, tokens=32, seqs=4, watermark=2)
    r.add(8, 4)                                    # 2 pages; nothing runs yet, so no watermark
    assert r.step() == [(0, 8)]
    r.add(12, 4)                                   # 3 pages would leave 1 < watermark 2
    r.add(2, 4)                                    # would fit, but must not overtake the head
    assert r.step() == [(0, 1)]
    assert [q.id for q in r.s.waiting] == [1, 2]


def test_policy_orders_admission():
    r = Rig(tokens=4, seqs=4, policy="srpt-aging", aging=0)
    r.add(30), r.add(3), r.add(9)
    assert r.step()[0] == (1, 3)                   # least remaining work first
    r2 = Rig(tokens=4, seqs=4, policy="fcfs")
    r2.add(30), r2.add(3)
    assert r2.step()[0] == (0, 4)
    # aging: a long request that has waited long enough overtakes a short newcomer
    r3 = Rig(tokens=4, seqs=1, policy="srpt-aging", aging=16)
    r3.add(4, 1)
    big = r3.add(40, 1)
    r3.step()                                      # request 0 runs and finishes; 1 waits
    r3.add(30, 1)
    assert r3.step()[0][0] == big.id               # 40 - 16*2 < 30 - 16*1


def test_when_pages_run_out_the_newest_is_preempted_and_recomputed_later():
    r = Rig(pages=4, tokens=16, seqs=4, watermark=0)
    a, b = r.add(7, 6), r.add(7, 6)
    assert r.step() == [(0, 7), (1, 7)]            # 2 pages each: the pool is full
    assert r.step() == [(0, 1), (1, 1)]            # 8 tokens each still fit
    got = r.step()                                 # a needs a third page: b, the newest, gives its pages back
    assert got == [(0, 1)] and b.state == SeqState.WAITING and b.num_computed == 0 and b.num_preemptions == 1
    assert len(b.tokens) == 9                      # prompt and generated tokens are kept
    assert r.s.num_preemptions == 1 and r.cache.num_free() == 1
    # b sits out the step in which it was preempted, then waits until a is done
    while a.state != SeqState.FINISHED:
        assert all(i == 0 for i, _ in r.step())
    assert r.step() == [(1, 9)]                    # recompute of prompt + generated, then it goes on
    while b.state != SeqState.FINISHED:
        r.step()
    assert b.num_generated == 6 and r.cache.num_free() == 4


def test_oldest_is_never_preempted_for_a_newer_one_and_a_lone_request_preempts_itself():
    r = Rig(pages=2, tokens=16, seqs=2, watermark=0)
    a = r.add(8, 2)
    assert r.step() == [(0, 8)]
    # a holds both pages and needs a third for its next token: no victim, nothing in flight -> it preempts itself
    assert r.step() == [] and a.num_preemptions == 1 and a.state == SeqState.WAITING


def test_a_full_pool_never_stalls_the_oldest():
    r = Rig(pages=4, tokens=8, seqs=2, watermark=0)
    a, b = r.add(14, 1), r.add(8, 1)
    assert r.step() == [(0, 8)]                    # a: 2 pages
    assert r.step() == [(0, 6)]                    # a's rest: the pool is full, b cannot be admitted
    for _ in range(20):
        if not r.s.has_work():
            break
        assert r.step() != [] or not r.s.has_work()
    assert not r.s.has_work() and r.cache.num_free() == 4 and a.num_preemptions == 0


def test_in_flight_batches_are_not_scheduled_again_and_abandon_gives_them_back():
    r = Rig(tokens=8)
    a = r.add(20, 2)
    b1 = r.s.schedule()
    assert [(q.id, n) for q, n in b1.seqs] == [(0, 8)]
    assert r.s.schedule().empty()                  # a is in flight
    r.cache.truncate(a.cache, a.num_computed)      # the step failed
    r.s.abandon(b1)
    assert r.cache.num_free() == 64
    assert [(q.id, n) for q, n in r.s.schedule().seqs] == [(0, 8)]


def test_cancel_while_waiting_running_or_preempted():
    r = Rig(pages=4, tokens=16, seqs=4, watermark=0)
    a, b, c = r.add(7, 6), r.add(7, 6), r.add(3, 2)
    r.step()
    r.finish(c)                                    # still waiting (no page was free for it)
    r.finish(b)                                    # running
    assert r.cache.num_free() == 2
    while r.s.has_work():
        r.step()
    assert a.num_generated == 6 and r.cache.num_free() == 4


def test_state_slots_are_taken_at_admission_and_admission_stops_when_none_is_left():
    """Requests that wait hold nothing, however many there are; a request gets its slot when it is admitted and
    loses it when it is preempted or ends; with no slot free admission stops (it does not raise)."""
    r = Rig(pages=64, tokens=32, seqs=4, slots=2)
    qs = [r.add(3, max_tokens=3) for _ in range(40)]
    assert r.states.num_free == 2 and all(q.cache.state_slot == -1 for q in qs)
    assert r.step() == [(0, 3), (1, 3)]                   # two slots: two requests run, although four are allowed
    assert r.states.num_free == 0 and {qs[0].cache.state_slot, qs[1].cache.state_slot} == {0, 1}
    assert r.step() == [(0, 1), (1, 1)]
    assert r.step() == [(0, 1), (1, 1)]                   # both end here and give their slots back
    assert r.states.num_free == 2
    assert r.step() == [(2, 3), (3, 3)]
    while r.s.has_work():
        r.step()
    assert all(q.num_generated == 3 for q in qs) and r.states.num_free == 2 and r.cache.num_free() == 64


def test_a_preempted_request_gives_its_state_slot_back():
    r = Rig(pages=4, tokens=16, seqs=4, watermark=0, slots=3)
    a, b = r.add(7, 6), r.add(7, 6)
    r.step(), r.step()
    assert r.states.num_free == 1
    assert r.step() == [(0, 1)] and b.state == SeqState.WAITING and b.cache.state_slot == -1
    assert r.states.num_free == 2
    while r.s.has_work():
        r.step()
    assert a.num_generated == b.num_generated == 6 and r.states.num_free == 3


@pytest.mark.parametrize("seed", range(300))
def test_randomized_simulation_keeps_the_invariants(seed):
    rng = random.Random(seed)
    needs = [CacheNeed("full", 1, 8)] + ([CacheNeed("window", 1, 8, window=rng.choice([6, 13]))] if seed % 3 == 0 else [])
    pages, tokens, seqs = rng.randint(6, 40), rng.choice([4, 8, 16, 32]), rng.randint(1, 4)
    r = Rig(pages=pages, tokens=max(tokens, seqs), seqs=seqs, policy=rng.choice(["fcfs", "srpt-aging"]),
            aging=rng.choice([0, 4, 16]), needs=needs, slots=rng.choice([None, 1, 2, 5]),
            window_requests=rng.choice([None, seqs]) if len(needs) > 1 else None)
    cap = pages * PAGE
    pending_adds = rng.randint(3, 12)
    empty_in_a_row = 0
    for step in range(4000):
        if pending_adds and rng.random() < 0.4:
            prompt = rng.randint(1, min(cap - 1, 50))
            r.add(prompt, max_tokens=min(rng.randint(1, 12), cap - prompt))
            pending_adds -= 1
        if rng.random() < 0.03:
            live = [q for q in r.seqs if q.state != SeqState.FINISHED]
            if live:
                r.finish(rng.choice(live))
        if not r.s.has_work():
            if not pending_adds:
                break
            continue
        oldest = r.s.running[0] if r.s.running else None
        before = oldest.num_preemptions if oldest else 0
        b = r.s.schedule()
        assert sum(n for _, n in b.seqs) <= r.s.config.serving.max_tokens_per_step
        assert len(b.seqs) <= seqs and len(r.s.running) <= seqs
        assert len({q.id for q, _ in b.seqs}) == len(b.seqs)
        for q, n in b.seqs:
            assert 0 < n <= q.num_pending
            assert len(q.cache.tables[0]) >= blocks_for(q.num_computed + n, PAGE)
        if oldest is not None and len(r.s.running) > 1 and oldest in r.s.running:
            assert oldest.num_preemptions == before, "the oldest running request was preempted for a newer one"
        empty_in_a_row = empty_in_a_row + 1 if b.empty() else 0
        assert empty_in_a_row <= 1, "two empty steps in a row: the scheduler stalled"
        r.finish_step(b)
        # between steps a table holds exactly the pages its computed tokens need; every page has one owner
        live = [q for q in r.seqs if q.state != SeqState.FINISHED]
        for g, pool in enumerate(r.cache.pools):
            held = [p for q in live for p in q.cache.tables[g].held()]
            assert len(held) == len(set(held)) and len(held) + pool.num_free == pool.num_blocks
        for q in live:
            assert len(q.cache.tables[0]) == blocks_for(q.num_computed, PAGE)
        if r.states is not None:
            # a slot has one owner, who runs; whoever waits holds none
            owned = [q.cache.state_slot for q in live if q.cache.state_slot >= 0]
            assert len(owned) == len(set(owned)) and len(owned) + r.states.num_free == r.states.max_requests
            assert all(q.cache.state_slot >= 0 for q in r.s.running if q.num_computed > 0)
            assert all(q.cache.state_slot == -1 for q in r.s.waiting)
    assert not r.s.has_work(), "not every request finished"
    assert all(q.state == SeqState.FINISHED for q in r.seqs)
    assert all(p.num_free == p.num_blocks for p in r.cache.pools)
    assert r.states is None or r.states.num_free == r.states.max_requests


def test_a_batch_that_is_neither_complete_nor_abandoned_keeps_its_requests_out_and_requeue_starts_one_over():
    """Requests of a batch in flight are skipped by the next decision until the engine calls `complete` (which it
    does at once when it decides the next step behind a step in flight) or `abandon`; `requeue` puts a request
    whose pages the engine took back into the waiting queue, wherever it was."""
    r = Rig(pages=16, tokens=16, seqs=4)
    a, b = r.add(6, max_tokens=100), r.add(3, max_tokens=100)
    batch = r.s.schedule()
    assert r.s._busy(a) and r.s._busy(b) and r.s.schedule().empty()
    r.finish_step(batch)
    assert not r.s._busy(a) and [(q.id, n) for q, n in r.s.schedule().seqs] == [(a.id, 1), (b.id, 1)]
    # the engine's part after a failed step whose bookkeeping had been moved on: pages back, computed again
    for q in (a, b):
        r.cache.reset(q.cache)
        q.num_computed = 0
    r.s.finish(b)                               # as for a request taken out because its last token was in flight
    r.s.requeue(a)
    r.s.requeue(b)
    assert a not in r.s.running and r.s.waiting == [a, b] and a.state == SeqState.WAITING and not r.s._busy(a)
    assert r.cache.num_free() == 16
    assert r.step() == [(a.id, 7), (b.id, 4)]      # prompt and the generated token again
