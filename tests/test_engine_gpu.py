"""Generation through the Python entry point and the scheduler, against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import assert_logits_close

pytestmark = pytest.mark.gpu


def engine_for(model_dir, dtype="float32", **kw):
    from tiny_inference_engine_b200 import load_engine
    return load_engine(model_dir, dtype=dtype, **kw)


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e", "tiny_b4"])
def test_greedy_and_sampled_generation_match_the_plain_implementation(tiny_models, name):
    from tiny_inference_engine_b200 import SamplingParams
    cfg, page, w, d = tiny_models[name]
    eng = engine_for(d, num_pages=64, page_size=page)
    rng = np.random.default_rng(2)
    for n_prompt in (1, 9, 40):
        prompt = rng.integers(0, cfg["vocab_size"], n_prompt).tolist()
        assert eng.generate(prompt, SamplingParams(max_tokens=8)) == plain.generate(w, cfg, prompt, 8)
        assert eng.generate(prompt, SamplingParams(max_tokens=6, temperature=0.8, seed=7)) == \
            plain.generate(w, cfg, prompt, 6, temperature=0.8, seed=7)
        assert eng.generate(prompt, SamplingParams(max_tokens=6, temperature=1.3, seed=3, top_k=10, top_p=0.9)) == \
            plain.generate(w, cfg, prompt, 6, temperature=1.3, seed=3, top_k=10, top_p=0.9)
    assert eng.cache.num_free() == 64 and not eng.has_work()


def test_bfloat16_generation_follows_the_plain_one_where_the_choice_is_clear(tiny_models):
    from tiny_inference_engine_b200 import SamplingParams
    cfg, page, w, d = tiny_models["tiny_b"]
    eng = engine_for(d, dtype="bfloat16", num_pages=64, page_size=page)
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()}
    checked = steps = 0
    for seed in (3, 4, 5):
        prompt = np.random.default_rng(seed).integers(0, cfg["vocab_size"], 20).tolist()
        got = eng.generate(prompt, SamplingParams(max_tokens=12))
        tokens = list(prompt)
        for t in got:                               # teacher-forced: each step's choice is checked on its own
            logits = plain.forward(wq, cfg, tokens)[-1]
            top = np.sort(logits)[-2:]
            steps += 1
            if top[1] - top[0] > 0.04 * np.abs(logits).max():
                assert t == int(np.argmax(logits))
                checked += 1
            tokens.append(t)
    assert checked >= steps // 2, f"only {checked} of {steps} steps had a clear choice: the test shows too little"


@pytest.mark.parametrize("pages", [256, 7])
@pytest.mark.parametrize("sampled", [False, True])
def test_batched_requests_generate_what_each_generates_alone(tiny_models, pages, sampled):
    """Eight mixed requests, 16 tokens per step, with plenty of pages and with so few that requests
    are preempted and recomputed; greedy and seeded temperature sampling (the reference's
    tests/engine/test_engine_batching.cpp:25-75)."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig
    cfg, page, w, d = tiny_models["tiny_b"]
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (1, 30, 7, 12, 3, 22, 9, 16)]
    params = [SamplingParams(max_tokens=4 + i, temperature=0.8 if sampled else 0.0, seed=100 + i) for i in range(8)]
    alone = engine_for(d, num_pages=64, page_size=page)
    want = [alone.generate(p, q) for p, q in zip(prompts, params)]
    eng = engine_for(d, num_pages=pages, page_size=page, serving=ServingConfig(16, 8), policy="fcfs")
    got = eng.generate_batch(prompts, params)
    assert got == want
    st = eng.stats()
    assert (st.preemptions > 0) == (pages == 7)
    assert eng.cache.num_free() == pages and st.steps > 0 and st.decode_tokens > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pages", [256, 9])
def test_steps_queued_ahead_change_no_token(tiny_models, dtype, pages):
    """With run_ahead the next decode step is queued before this one's tokens are read and takes them
    from the device. Same tokens as without, for requests that end by length, by a stop token (one step
    runs in vain) and at different times, with plenty of pages and with so few that requests are
    preempted; no page is lost."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig
    cfg, page, w, d = tiny_models["tiny_b"]
    rng = np.random.default_rng(14)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (3, 17, 8, 25, 1, 11)]
    params = [SamplingParams(max_tokens=5 + 4 * i, temperature=0.7 if i % 2 else 0.0, seed=50 + i) for i in range(6)]
    plain_run = engine_for(d, dtype=dtype, num_pages=64, page_size=page, serving=ServingConfig(16, 8, run_ahead=False))
    free_run = plain_run.generate_batch(prompts, params)
    stop = [free_run[3][6], free_run[5][10]]              # tokens that two of the requests do generate
    outs = {}
    for ahead in (False, True):
        eng = engine_for(d, dtype=dtype, num_pages=pages, page_size=page, stop_tokens=stop, policy="fcfs",
                         serving=ServingConfig(16, 8, run_ahead=ahead))
        outs[ahead] = eng.generate_batch(prompts, params)
        st = eng.stats()
        assert (st.steps_ahead > 0) == ahead
        while eng.has_work():                               # a step may still be queued for requests that have ended
            eng.step()
        assert eng.cache.num_free() == pages
        assert st.decode_tokens > 0 and (st.preemptions > 0) == (pages == 9)
    assert outs[True] == outs[False]
    assert any(len(o) < p.max_tokens for o, p in zip(outs[True], params)), "no request was stopped by a stop token"
    # one request alone, through generate(), ended by a stop token while a step is queued ahead; then the next one
    eng = engine_for(d, dtype=dtype, num_pages=64, page_size=page, stop_tokens=[free_run[1][5]])
    assert eng.generate(prompts[1], params[1]) == free_run[1][:free_run[1].index(free_run[1][5]) + 1]
    assert eng.generate(prompts[2], params[2]) == plain_run.generate(prompts[2], params[2])
    assert eng.stats().steps_ahead > 0


@pytest.mark.timeout(300)
def test_mixed_steps_at_full_width_with_wide_layers(tmp_path):
    """Layers as wide as Qwen3-8B's (two of them, random weights), 512 tokens a step, sixteen requests at once:
    steps that mix two prompt portions with decoded tokens run the matrix products on pairs of SMs beside the
    decode kernels. Three runs give the same tokens with and without steps queued ahead, and nothing is lost."""
    import json

    from tiny_inference_engine_b200 import (Engine, SamplingParams, Scheduler, SchedulerConfig, ServingConfig, StepRunner,
                                            load_model, make_cache)
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 32000, "hidden_size": 4096,
           "intermediate_size": 12288, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8,
           "head_dim": 128, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
           "tie_word_embeddings": False}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    model = load_model(str(tmp_path), "bfloat16", random_weights=True, seed=0)
    rng = np.random.default_rng(1)
    reqs = [(rng.integers(0, 32000, int(rng.integers(1, 700))).tolist(),
             SamplingParams(max_tokens=40 + 5 * i, temperature=[0.0, 0.9][i % 2], seed=i)) for i in range(16)]
    outs = []
    for ahead in (False, True, True):
        cache, states = make_cache(model, page_size=16, num_pages=1200, max_requests=32)
        serving = ServingConfig(512, 16, run_ahead=ahead)
        runner = StepRunner(model, cache, 512, 16, 16, states=states)
        eng = Engine(model, cache, Scheduler(cache, SchedulerConfig(serving=serving, policy="fcfs")), serving, states=states,
                     runner=runner)
        outs.append(eng.generate_batch([p for p, _ in reqs], [q for _, q in reqs]))
        while eng.has_work():
            eng.step()
        assert cache.num_free() == 1200 and eng.stats().prefill_tokens == sum(len(p) for p, _ in reqs)
        assert (eng.stats().steps_ahead > 0) == ahead
    assert outs[0] == outs[1] == outs[2]
    assert all(len(o) == q.max_tokens for o, (_, q) in zip(outs[0], reqs))


def test_a_failed_step_is_rolled_back_and_the_requests_still_finish(tiny_models):
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig
    cfg, page, w, d = tiny_models["tiny_a"]
    prompts = [[5, 6, 7, 8, 9, 10, 11, 12, 13], [3] * 20, [200, 100]]
    alone = engine_for(d, num_pages=64, page_size=page)
    want = [alone.generate(p, SamplingParams(max_tokens=6)) for p in prompts]
    eng = engine_for(d, num_pages=64, page_size=page, serving=ServingConfig(8, 4), policy="fcfs")
    calls = {"n": 0}

    def fail_third(ctx):
        calls["n"] += 1
        if calls["n"] == 3:
            raise RuntimeError("injected")

    eng.runner.fail_hook = fail_third
    ids = [eng.add_request(p, SamplingParams(max_tokens=6)) for p in prompts]
    failures = 0
    while eng.has_work():
        try:
            eng.step()
        except RuntimeError:
            failures += 1
    assert failures == 1
    assert [eng.sequence(i).tokens[eng.sequence(i).prompt_len:] for i in ids] == want
    assert eng.cache.num_free() == 64


def test_tiny_a_workload_as_the_reference_engine_ran_it(tmp_path):
    """tiny-A: prompts of 5, 17 and 33 tokens, greedy, 8 new tokens each, 8 tokens a step, pages of 16, first come
    first served. The reference's own Engine ran exactly this (tests/golden/make_golden.py); the ids are its ids."""
    from test_plain import golden_requests, golden_tokens
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig
    plain.write_model_dir(tmp_path, plain.TINY_A, plain.random_weights(plain.TINY_A, 0))
    reqs = golden_requests("tiny_a")
    assert [(len(p), n) for n, p in reqs] == [(5, 8), (17, 8), (33, 8)]
    for run_ahead in (False, True):
        eng = engine_for(tmp_path, num_pages=256, page_size=16, serving=ServingConfig(8, 8, run_ahead=run_ahead), policy="fcfs")
        got = eng.generate_batch([p for _, p in reqs], [SamplingParams(max_tokens=n) for n, _ in reqs])
        assert got == golden_tokens("tiny_a")
        assert eng.stats().seqs_scheduled > eng.stats().steps          # really batched
        assert eng.stats().prefill_tokens == 5 + 17 + 33 and eng.cache.num_free() == 256


def test_tiny_b_workload_with_a_pool_that_forces_a_preemption(tmp_path):
    """tiny-B (4 query heads over one kv head, head 32, q width 128 beside a hidden size of 96, untied output table,
    theta 1e6, eps 1e-5): prompts of 1, 9, 40 and 64 tokens, 6 new tokens each, 13 tokens a step, pages of 8, and a pool
    of so few pages that a request is preempted and computed again. Greedy: the ids of the reference's own Engine,
    which preempted too. Temperature 0.8 with Philox seed 7 (the reference draws from mt19937, so no reference ids):
    what every request generates alone, and what the plain implementation generates."""
    from test_plain import GOLDEN, golden_requests, golden_tokens
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, load_engine
    cfg = plain.TINY_B4
    w = plain.random_weights(cfg, 1)
    plain.write_model_dir(tmp_path, cfg, w)
    reqs = golden_requests("tiny_b4")
    assert [(len(p), n) for n, p in reqs] == [(1, 6), (9, 6), (40, 6), (64, 6)]
    pool = int((GOLDEN / "tiny_b4_small_pool.txt").read_text())
    prompts = [p for _, p in reqs]

    def small_engine(run_ahead):
        # as the reference ran it: first come first served, and admission may use the last free page
        return load_engine(tmp_path, dtype="float32", num_pages=pool, page_size=8, policy="fcfs", watermark_pages=0,
                           serving=ServingConfig(13, 8, run_ahead=run_ahead))

    for run_ahead in (False, True):
        eng = small_engine(run_ahead)
        assert eng.generate_batch(prompts, [SamplingParams(max_tokens=n) for n, _ in reqs]) == golden_tokens("tiny_b4", small=True)
        assert eng.stats().preemptions >= 1 and eng.cache.num_free() == pool
        sampled = [SamplingParams(max_tokens=n, temperature=0.8, seed=7) for n, _ in reqs]
        got = small_engine(run_ahead).generate_batch(prompts, sampled)
        alone = engine_for(tmp_path, num_pages=64, page_size=8)
        assert got == [alone.generate(p, q) for p, q in zip(prompts, sampled)]
        assert got == [plain.generate(w, cfg, p, 6, temperature=0.8, seed=7) for p in prompts]


@pytest.mark.parametrize("run_ahead", [False, True])
def test_a_nan_among_the_logits_ends_that_request_with_an_error_and_the_others_go_on(tiny_models, run_ahead):
    """A layer hook writes a NaN into the rows at position 12, which only the second request reaches: its row of
    logits cannot be sampled, the kernels say so with the ids, and the engine ends it as the reference does
    (src/sampling/sampler.cpp:18-26, src/engine/engine.cpp:157-174). The others generate what they generate alone."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig
    from tiny_inference_engine_b200.engine import FinishReason
    cfg, page, w, d = tiny_models["tiny_a"]
    prompts = [[5, 6, 7], [30, 31, 32, 33, 34, 35, 36, 37, 38], [200, 100], [9]]
    params = [SamplingParams(max_tokens=6, temperature=t, seed=4, top_k=k) for t, k in [(0.0, 0), (0.8, 0), (0.8, 5), (0.0, 0)]]
    alone = engine_for(d, num_pages=64, page_size=page)
    want = [alone.generate(p, q) for p, q in zip(prompts, params)]
    eng = engine_for(d, num_pages=64, page_size=page, serving=ServingConfig(16, 4, run_ahead=run_ahead), policy="fcfs")
    seen = {}
    eng.runner.fail_hook = lambda ctx: seen.__setitem__("ctx", ctx)      # called with every step's context; never fails

    def poison(layer, x, pending):
        if layer == 0:
            ctx = seen["ctx"]
            x[:ctx.T].masked_fill_((ctx.positions[:ctx.T] == 12)[:, None], float("nan"))

    eng.runner.layer_hook = poison
    ids = [eng.add_request(p, q) for p, q in zip(prompts, params)]
    while eng.has_work():
        eng.step()
    seqs = [eng.sequence(i) for i in ids]
    # position 12 is the input of request 1's fifth generated token: four tokens came out
    assert seqs[1].finish_reason == FinishReason.ERROR and seqs[1].tokens[9:] == want[1][:4]
    for i in (0, 2, 3):
        assert seqs[i].finish_reason == FinishReason.LENGTH and seqs[i].tokens[len(prompts[i]):] == want[i]
    assert eng.cache.num_free() == 64 and all(t >= 0 for q in seqs for t in q.tokens)


@pytest.mark.parametrize("run_ahead", [False, True])
def test_a_mixer_with_state_of_its_own_under_the_engine_with_preemption_and_a_failed_step(run_ahead):
    """The running-mean toy mixer (state in the engine's state slots) under the scheduler: eight requests, three
    slots and a pool so small that requests are preempted, one step that fails, steps queued ahead or not. A request
    takes its slot when it is admitted and loses it when it is preempted; after a failed step requests with state
    start over. Every request generates what the plain restatement generates for it alone."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, StepRunner, make_cache
    from tiny_inference_engine_b200.engine import Engine, Scheduler, SchedulerConfig
    from tiny_inference_engine_b200.parts import Model
    from test_parts_gpu import DictSource
    from toy_parts import running_mean_model
    spec, w, cfg, plain_forward = running_mean_model()
    model = Model(spec, torch.float32).load(DictSource(w))
    serving = ServingConfig(16, 4, run_ahead=run_ahead)
    cache, states = make_cache(model, page_size=8, num_pages=6, max_requests=3)
    assert cache.needs_state_slot and states.bytes_per_slot == 4 * cfg["hidden_size"]
    runner = StepRunner(model, cache, serving.max_tokens_per_step, serving.max_seqs, serving.max_seqs, states=states)
    eng = Engine(model, cache, Scheduler(cache, SchedulerConfig(serving, policy="fcfs", watermark_pages=0)), serving,
                 states=states, runner=runner)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, 256, n).tolist() for n in (5, 17, 9, 1, 12, 3, 20, 7)]
    new = [10, 6, 12, 9, 5, 11, 4, 8]

    def plain_generate(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(plain_forward(toks)[-1].argmax()))
        return toks[len(prompt):]

    want = [plain_generate(p, n) for p, n in zip(prompts, new)]
    calls = {"n": 0}

    def fail_sixth(ctx):
        calls["n"] += 1
        if calls["n"] == 6:
            raise RuntimeError("injected")

    runner.fail_hook = fail_sixth
    ids = [eng.add_request(p, SamplingParams(max_tokens=n)) for p, n in zip(prompts, new)]
    assert states.num_free == 3                        # eight requests wait; none holds a slot
    failures = 0
    while eng.has_work():
        try:
            eng.step()
        except RuntimeError:
            failures += 1
    assert failures == 1 and eng.stats().preemptions >= 1
    assert [eng.sequence(i).tokens[len(p):] for i, p in zip(ids, prompts)] == want
    assert states.num_free == 3 and cache.num_free() == 6


def test_decode_steps_of_a_model_with_state_are_captured_when_its_mixer_says_it_can_be():
    """A mixer with state that reads the step through device tensors only says `graph_safe`; its model's decode steps
    then run as CUDA graphs (with sequences that pad a batch, whose state slot is -1), and the tokens are those of
    the plain restatement. The toy of the other tests reads the step on the host: its model stays out of graphs."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, StepRunner, make_cache
    from tiny_inference_engine_b200.engine import Engine, Scheduler, SchedulerConfig
    from tiny_inference_engine_b200.parts import Model
    from test_parts_gpu import DictSource
    from toy_parts import running_mean_model
    for on_device in (True, False):
        spec, w, cfg, plain_forward = running_mean_model(on_device=on_device)
        model = Model(spec, torch.float32).load(DictSource(w))
        serving = ServingConfig(16, 4)
        cache, states = make_cache(model, page_size=8, num_pages=32, max_requests=8)
        runner = StepRunner(model, cache, serving.max_tokens_per_step, serving.max_seqs, serving.max_seqs, states=states)
        assert runner.use_graphs == on_device
        eng = Engine(model, cache, Scheduler(cache, SchedulerConfig(serving, policy="fcfs")), serving, states=states, runner=runner)
        rng = np.random.default_rng(11)
        prompts = [rng.integers(0, 256, n).tolist() for n in (6, 1, 11)]           # three requests: a batch of four is padded
        got = eng.generate_batch(prompts, SamplingParams(max_tokens=9))
        for p, g in zip(prompts, got):
            toks = list(p)
            for t in g:
                assert t == int(plain_forward(toks)[-1].argmax())
                toks.append(t)
        assert (runner.graph_replays > 0) == on_device and states.num_free == 8


def test_capacity_errors_cancel_and_callbacks(tiny_models):
    from tiny_inference_engine_b200 import CapacityError, InvalidArgument, SamplingParams
    from tiny_inference_engine_b200.engine import FinishReason, SeqState
    cfg, page, w, d = tiny_models["tiny_a"]
    eng = engine_for(d, num_pages=4, page_size=page, stop_tokens=[])
    with pytest.raises(CapacityError, match="raise --kv-mem"):
        eng.add_request([1] * 64)
    with pytest.raises(CapacityError, match="context"):
        eng.add_request([1] * 512)
    with pytest.raises(InvalidArgument, match="outside vocabulary"):
        eng.add_request([1, 256])
    with pytest.raises(InvalidArgument, match="empty"):
        eng.add_request([])
    a = eng.add_request([1, 2, 3], SamplingParams(max_tokens=500))
    assert eng.sequence(a).params.max_tokens == 4 * page - 3      # clamped to the pool
    seen = []
    eng.set_token_callback(lambda i, t: (seen.append((i, t)), eng.cancel(i) if len(seen) == 3 else None))
    while eng.has_work():
        eng.step()
    assert len(seen) == 3 and eng.sequence(a).finish_reason == FinishReason.CANCELLED
    assert eng.cache.num_free() == 4
    eng.release(a)
    with pytest.raises(InvalidArgument, match="no sequence"):
        eng.sequence(a)
    # a stop token ends a request and is part of its output
    eng.set_token_callback(None)
    first = eng.generate([9, 9, 9], SamplingParams(max_tokens=5))
    eng2 = engine_for(d, num_pages=4, page_size=page, stop_tokens=[first[1]])
    assert eng2.generate([9, 9, 9], SamplingParams(max_tokens=5)) == first[:first.index(first[1]) + 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(tiny_models, dtype):
    """One token from position 0 on, then 600 more one by one (the split attention kernel sees one,
    two and three splits); all logits against the plain implementation."""
    from tiny_inference_engine_b200 import StepEntry, StepRunner, load_model, make_cache
    cfg, page, w, d = tiny_models["tiny_d" if dtype == "bfloat16" else "tiny_c"]   # bfloat16: the tensor-core kernels
    toks = np.random.default_rng(6).integers(0, cfg["vocab_size"], 601).tolist()
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    want = plain.forward(wq, cfg, toks)
    model = load_model(d, dtype)
    cache, states = make_cache(model, page_size=page, num_pages=40, max_requests=2)
    runner = StepRunner(model, cache, 64, 2, 8, states=states)
    req = cache.new_request()
    got = []
    for t, tok in enumerate(toks):
        assert cache.reserve(req, t + 1)
        got.append(runner.run([StepEntry(req, [tok], t, [0])]))
        if t % 50 == 0:
            got[-1] = got[-1].clone()
        got[-1] = got[-1].float().cpu().numpy()
    got = np.concatenate(got)
    assert_logits_close(got[:3], want[:3], dtype, "the first tokens")
    assert_logits_close(got, want, dtype, "600 decoded tokens")


def test_decode_graphs_at_a_context_in_the_last_bucket_of_the_block_table(tmp_path):
    """A model whose longest request has 40 pages (no power of two): max_seqs requests decode as one captured graph while
    one of them is at a context of 38 pages. The graph's table length is the next power of two, 64, capped at the 40
    the index buffer was sized for: the step fits, and its logits are the plain ones."""
    from tiny_inference_engine_b200 import StepEntry, StepRunner, load_model, make_cache
    cfg = dict(plain.TINY_A, max_position_embeddings=320)
    w = sharp_weights_for(cfg)
    plain.write_model_dir(tmp_path, cfg, w)
    model = load_model(tmp_path, "float32")
    page, seqs = 8, 4
    cache, states = make_cache(model, page_size=page, num_pages=40 + 3 * 6 + 2, max_requests=seqs)
    runner = StepRunner(model, cache, 320, seqs, seqs, states=states)
    assert runner._table_cap == 40
    rng = np.random.default_rng(12)
    lengths = [300, 9, 33, 41]
    toks = [rng.integers(0, cfg["vocab_size"], n + 3).tolist() for n in lengths]
    reqs = [cache.new_request() for _ in lengths]
    for r, t, n in zip(reqs, toks, lengths):
        assert cache.reserve(r, n + 3)
        runner.run([StepEntry(r, t[:n], 0, [])])
    want = [plain.forward(w, cfg, t) for t in toks]
    for step in range(3):
        out = runner.run([StepEntry(r, [t[n + step]], n + step, [0]) for r, t, n in zip(reqs, toks, lengths)]).float().cpu().numpy()
        for i, n in enumerate(lengths):
            assert_logits_close(out[i:i + 1], want[i][n + step:n + step + 1], "float32", f"request {i}, step {step}")
    assert runner.graph_replays >= 1 and all(key[1] == 40 for key in runner._graphs)


def sharp_weights_for(cfg):
    from conftest import sharp_weights
    return sharp_weights(cfg, 5)


def test_command_line_generates_the_plain_tokens(tiny_models):
    import subprocess
    import sys
    from conftest import ROOT
    cfg, page, w, d = tiny_models["tiny_a"]
    prompt = [7, 200, 13, 99, 5]
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "tie"), "generate", "-m", str(d), "-p", " ".join(map(str, prompt)),
                        "--dtype", "float32", "--temp", "0", "--top-k", "0", "--top-p", "1", "--max-tokens", "6", "--kv-mem", "1M"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [int(t) for t in r.stdout.split()] == plain.generate(w, cfg, prompt, 6)
    assert "[tie] cuda | load" in r.stderr and "6 tok generated" in r.stderr
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "tie"), "generate", "-m", str(d), "-p", "1 2 999"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 1 and "outside vocabulary" in r.stderr
