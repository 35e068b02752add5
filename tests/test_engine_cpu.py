"""The engine's decisions without a GPU: a stand-in for the step function (tests/fake_runner.py) whose tokens depend
on a request's whole prefix, so that any token fed at a wrong position, taken from a wrong row, sampled with a wrong
index, lost in a preemption or handed out twice changes what a request generates. Every run is compared with what
each request generates alone."""
import random

import pytest

import torch

from fake_runner import VOCAB, FakeRunner, generate_alone
from tiny_inference_engine_b200.cache import CacheManager, StateSlots
from tiny_inference_engine_b200.engine import Engine, FinishReason, Scheduler, SchedulerConfig, SeqState, ServingConfig
from tiny_inference_engine_b200.parts import CacheNeed, StateNeed
from tiny_inference_engine_b200.sampling import SamplingParams

PAGE = 4


class _Spec:
    vocab_size = VOCAB
    max_positions = 4096


class _Model:
    spec = _Spec()


def make_engine(pages=64, tokens=16, seqs=4, policy="fcfs", run_ahead=True, stop=(), slots=None):
    """With `slots` the stand-in model keeps per-request state (a count of the tokens run) in that many slots."""
    states = StateSlots([StateNeed((1,), torch.int64)], slots, device="cpu") if slots else None
    cache = CacheManager([CacheNeed("full", 1, 8)], page_size=PAGE, num_pages=pages, state_slots=states)
    serving = ServingConfig(tokens, seqs, run_ahead=run_ahead)
    runner = FakeRunner(cache, tokens, seqs, states=states)
    return Engine(_Model(), cache, Scheduler(cache, SchedulerConfig(serving, policy)), serving, stop_tokens=stop,
                  states=states, runner=runner)


def drain(eng):
    while eng.has_work():
        eng.step()


@pytest.mark.parametrize("run_ahead", [False, True])
def test_batched_requests_generate_what_each_generates_alone(run_ahead):
    prompts = [[1, 2, 3], list(range(30)), [7] * 9, [5], list(range(100, 121))]
    params = [SamplingParams(max_tokens=4 + 3 * i, seed=i) for i in range(5)]
    eng = make_engine(run_ahead=run_ahead)
    assert eng.generate_batch(prompts, params) == [generate_alone(p, q) for p, q in zip(prompts, params)]
    drain(eng)
    assert eng.cache.num_free() == 64
    assert (eng.stats().steps_ahead > 0) == run_ahead
    assert eng.stats().prefill_tokens == sum(map(len, prompts))
    assert eng.stats().decode_tokens == sum(q.max_tokens for q in params) - len(prompts)


@pytest.mark.parametrize("slots", [None, 3, 16])
def test_ten_times_more_requests_than_a_step_holds_wait_at_no_cost_and_all_finish(slots):
    """A request that waits holds no page and no state slot (src/engine/sequence.h:15-30,
    src/engine/engine.cpp:51-62: add_request allocates nothing), so the queue is as long as one likes."""
    rng = random.Random(5)
    eng = make_engine(pages=24, tokens=16, seqs=4, slots=slots)
    prompts = [[rng.randrange(VOCAB) for _ in range(rng.randint(1, 20))] for _ in range(40)]
    params = [SamplingParams(max_tokens=rng.randint(1, 9), seed=i) for i in range(40)]
    ids = [eng.add_request(p, q) for p, q in zip(prompts, params)]
    assert eng.cache.num_free() == 24 and (slots is None or eng.states.num_free == slots)
    drain(eng)
    assert [eng.sequence(i).tokens[eng.sequence(i).prompt_len:] for i in ids] == \
        [generate_alone(p, q) for p, q in zip(prompts, params)]
    assert eng.cache.num_free() == 24 and (slots is None or eng.states.num_free == slots)


@pytest.mark.parametrize("run_ahead", [False, True])
def test_a_row_the_sampler_refuses_ends_its_request_with_an_error_and_the_others_go_on(run_ahead):
    """A NaN among the logits, or nothing finite: the reference's sampler raises and the engine ends that request
    with FinishReason::Error while the step's other requests get their tokens
    (src/sampling/sampler.cpp:18-26, src/engine/engine.cpp:157-174)."""
    from fake_runner import UNSAMPLABLE
    prompts = [[1, 2, 3], [4, 5, 6, 7, 8, 9, 10, 11, 12], [13], [14, 15]]
    q = SamplingParams(max_tokens=8, seed=2)
    want = [generate_alone(p, q) for p in prompts]
    eng = make_engine(run_ahead=run_ahead)
    bad = prompts[1] + want[1][:3]                 # request 1's fourth token cannot be sampled
    eng.runner.refuse = lambda prefix: prefix == bad
    seen = []
    eng.set_token_callback(lambda i, t: seen.append(t))
    ids = [eng.add_request(p, q) for p in prompts]
    drain(eng)
    seqs = [eng.sequence(i) for i in ids]
    assert seqs[1].finish_reason == FinishReason.ERROR and seqs[1].tokens[len(prompts[1]):] == want[1][:3]
    for i in (0, 2, 3):
        assert seqs[i].finish_reason == FinishReason.LENGTH and seqs[i].tokens[len(prompts[i]):] == want[i]
    assert UNSAMPLABLE not in seen and all(t >= 0 for s in seqs for t in s.tokens)
    assert eng.cache.num_free() == 64


@pytest.mark.parametrize("seed", range(120))
def test_random_workloads_with_small_pools_stop_tokens_and_cancels(seed):
    rng = random.Random(seed)
    n = rng.randint(2, 9)
    prompts = [[rng.randrange(VOCAB) for _ in range(rng.randint(1, 40))] for _ in range(n)]
    params = [SamplingParams(max_tokens=rng.randint(1, 30), seed=rng.randrange(100)) for _ in range(n)]
    free = [generate_alone(p, q) for p, q in zip(prompts, params)]
    stop = {rng.choice(rng.choice(free)) for _ in range(2)} if rng.random() < 0.6 else set()
    want = [generate_alone(p, q, stop) for p, q in zip(prompts, params)]
    longest = max(len(p) + q.max_tokens for p, q in zip(prompts, params))
    pages = rng.choice([-(-longest // PAGE) + 1, 24, 200])
    eng = make_engine(pages=pages, tokens=rng.choice([8, 16, 64]), seqs=rng.choice([2, 4, 8]), run_ahead=rng.random() < 0.7,
                      policy=rng.choice(["fcfs", "srpt-aging"]), stop=stop, slots=rng.choice([None, None, 2, 5, 16]))
    ids, arrivals = [], sorted(rng.randint(0, 12) for _ in range(n))
    cancel_at = {i: rng.randint(1, 5) for i in range(n) if rng.random() < 0.15}    # request -> after how many of its tokens
    seen = {}

    def on_token(seq_id, token):
        seen.setdefault(seq_id, []).append(token)
        i = ids.index(seq_id)
        if cancel_at.get(i) == len(seen[seq_id]):
            eng.cancel(seq_id)

    eng.set_token_callback(on_token)
    step = 0
    while len(ids) < n or eng.has_work():
        while len(ids) < n and arrivals[len(ids)] <= step:
            ids.append(eng.add_request(prompts[len(ids)], params[len(ids)]))
        eng.step()
        step += 1
        assert step < 5000
    for i, sid in enumerate(ids):
        seq = eng.sequence(sid)
        got = seq.tokens[seq.prompt_len:]
        assert seq.state == SeqState.FINISHED and seen.get(sid, []) == got
        if i in cancel_at and cancel_at[i] <= len(want[i]):      # its own callback cancelled it, even at its last token
            assert seq.finish_reason == FinishReason.CANCELLED and got == want[i][:cancel_at[i]]
        else:
            assert got == want[i], f"request {i}"
            assert seq.finish_reason == (FinishReason.STOP if got[-1] in stop else FinishReason.LENGTH)
    assert eng.cache.num_free() == pages
    assert eng.states is None or eng.states.num_free == eng.states.max_requests


@pytest.mark.parametrize("slots", [None, 4])
@pytest.mark.parametrize("run_ahead", [False, True])
@pytest.mark.parametrize("at_read", [False, True])
@pytest.mark.parametrize("fail_at", [1, 2, 3, 5, 8, 9, 10, 13])
def test_a_failed_step_is_rolled_back(run_ahead, fail_at, at_read, slots):
    """A step that fails while it is being queued, or whose ids cannot be read (with another step already queued behind
    it): the engine raises once, and every request still generates what it generates alone. Requests with state of
    fixed size start over instead of being cut back, since that state cannot be cut back."""
    prompts = [list(range(9)), [3] * 20, [200, 100], [9, 8, 7, 6]]
    params = [SamplingParams(max_tokens=7, seed=i) for i in range(4)]
    eng = make_engine(tokens=8, seqs=4, run_ahead=run_ahead, slots=slots)
    if at_read:
        eng.runner.fail_read_at = {fail_at}
    else:
        eng.runner.fail_at = {fail_at}
    ids = [eng.add_request(p, q) for p, q in zip(prompts, params)]
    failures = 0
    while eng.has_work():
        try:
            eng.step()
        except RuntimeError:
            failures += 1
    assert failures == (1 if eng.runner.runs >= fail_at else 0) and eng.runner.runs >= 8
    assert [eng.sequence(i).tokens[eng.sequence(i).prompt_len:] for i in ids] == [generate_alone(p, q) for p, q in zip(prompts, params)]
    assert eng.cache.num_free() == 64


def test_generate_one_after_another_with_a_step_still_queued_for_the_one_that_stopped():
    """generate() returns as soon as its request has ended; the step that was queued behind its last one is dealt with
    by the next call, and the next request starts from a clean pool."""
    p1, p2 = [5, 6, 7, 8], list(range(40, 70))
    q = SamplingParams(max_tokens=12, seed=3)
    free = generate_alone(p1, q)
    eng = make_engine(stop={free[4]})
    assert eng.generate(p1, q) == free[:5]
    assert eng._ahead is not None            # a step runs in vain for it
    assert eng.generate(p2, q) == generate_alone(p2, q, {free[4]})
    drain(eng)
    assert eng.cache.num_free() == 64 and eng.stats().steps_ahead > 0


def test_requests_that_cannot_run_are_refused_and_max_tokens_is_clamped():
    from tiny_inference_engine_b200.errors import CapacityError, InvalidArgument
    eng = make_engine(pages=4)
    with pytest.raises(CapacityError, match="raise --kv-mem"):
        eng.add_request([1] * 16)
    with pytest.raises(InvalidArgument, match="outside vocabulary"):
        eng.add_request([1, VOCAB])
    with pytest.raises(InvalidArgument, match="empty"):
        eng.add_request([])
    a = eng.add_request([1, 2, 3], SamplingParams(max_tokens=500))
    assert eng.sequence(a).params.max_tokens == 4 * PAGE - 3          # what the pool can hold
    drain(eng)
    seq = eng.sequence(a)
    assert seq.finish_reason == FinishReason.LENGTH and seq.tokens[3:] == generate_alone([1, 2, 3], seq.params)
    with pytest.raises(InvalidArgument, match="still running|no sequence"):
        eng.release(99)
    eng.release(a)
    assert eng.cache.num_free() == 4


def test_a_callback_that_raises_ends_the_requests_that_were_to_get_a_token_and_the_engine_goes_on():
    prompts = [[1, 2], [3, 4, 5], [6]]
    q = SamplingParams(max_tokens=6, seed=1)
    eng = make_engine()
    ids = [eng.add_request(p, q) for p in prompts]
    calls = []

    def on_token(seq_id, token):
        calls.append(seq_id)
        if len(calls) == 4:
            raise ValueError("from the callback")

    eng.set_token_callback(on_token)
    with pytest.raises(ValueError):
        drain(eng)
    eng.set_token_callback(None)
    drain(eng)
    states = [eng.sequence(i) for i in ids]
    assert all(s.state == SeqState.FINISHED for s in states) and eng.cache.num_free() == 64
    assert any(s.finish_reason == FinishReason.ERROR for s in states)
    assert all(-1 not in s.tokens for s in states)                     # no placeholder is left behind
    b = eng.add_request([9, 9], q)
    drain(eng)
    assert eng.sequence(b).tokens[2:] == generate_alone([9, 9], q)
