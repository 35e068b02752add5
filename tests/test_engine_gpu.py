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


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b", "tiny_c", "tiny_d", "tiny_e"])
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
    prompt = np.random.default_rng(3).integers(0, cfg["vocab_size"], 20).tolist()
    got = eng.generate(prompt, SamplingParams(max_tokens=12))
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()}
    tokens = list(prompt)
    for t in got:                                   # teacher-forced: each step's choice is checked on its own
        logits = plain.forward(wq, cfg, tokens)[-1]
        top = np.sort(logits)[-2:]
        if top[1] - top[0] > 0.04 * np.abs(logits).max():
            assert t == int(np.argmax(logits))
        tokens.append(t)


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
