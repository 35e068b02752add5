"""Layers built alike issued by one call (ops/replay.py, csrc/layer_replay.cu) against the same layers issued
one by one from Python: the same launchers with the same arguments, so every logit must be the same bit for
bit, in steps of every kind (a whole prompt, portions, portions beside decoded tokens, decoding with and without
captured graphs), in both dtypes; and against the plain implementation, so that a layer given another layer's
weights or cache planes would show."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from conftest import assert_logits_close, sharp_weights

pytestmark = pytest.mark.gpu


def _steps(model, cfg, page, graphs, prompts):
    """A fixed script of steps over three requests; returns the logits of every step that wanted some."""
    from tiny_inference_engine_b200 import StepEntry, StepRunner, make_cache
    cache, states = make_cache(model, page_size=page, num_pages=64, max_requests=8)
    runner = StepRunner(model, cache, 256, 8, 256, states=states, use_graphs=graphs)
    a, b, c = (cache.new_request() for _ in range(3))
    pa, pb, pc = prompts
    for r, p in ((a, pa), (b, pb), (c, pc)):
        assert cache.reserve(r, len(p) + 8)
    out = []

    def run(entries):
        got = runner.run(entries)
        if got is not None:
            out.append(got.float().cpu().numpy().copy())

    run([StepEntry(a, pa[:150], 0, list(range(150)))])                                  # a whole prompt, every row
    run([StepEntry(b, pb[:20], 0, [19])])                                               # portions
    run([StepEntry(b, pb[20:37], 20, [0, 16]), StepEntry(a, pa[150:151], 150, [0])])    # a portion beside a decoded token
    run([StepEntry(c, pc[:2], 0, []), StepEntry(a, pa[151:152], 151, [0]), StepEntry(b, pb[37:38], 37, [0])])
    run([StepEntry(c, pc[2:131], 2, [128])])
    for i in range(4):                                                                  # decoding: graphs if asked for
        run([StepEntry(a, pa[152 + i:153 + i], 152 + i, [0]), StepEntry(b, pb[38 + i:39 + i], 38 + i, [0]),
             StepEntry(c, pc[131 + i:132 + i], 131 + i, [0])])
    torch.cuda.synchronize()
    runner.check()
    return out


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype,base,page", [("bfloat16", "TINY_D", 16), ("float32", "TINY_B", 8), ("bfloat16", "TINY_E", 16)])
def test_layers_issued_by_one_call_give_the_same_bits(tmp_path, dtype, base, page, graphs):
    from tiny_inference_engine_b200 import load_model
    from tiny_inference_engine_b200.ops import replay
    cfg = dict(getattr(plain, base), num_hidden_layers=6)
    w = sharp_weights(cfg, 5)
    plain.write_model_dir(tmp_path, cfg, w)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (156, 42, 135)]
    results = {}
    for on in (False, True):
        model = load_model(tmp_path, dtype)
        assert model.layer_replay
        model.layer_replay = on
        before = replay.layers_repeated
        results[on] = _steps(model, cfg, page, graphs, prompts)
        repeated = replay.layers_repeated - before
        # Six layers alike: after the first two of a forward the other four go through the list; not in the
        # model's first forward, and a replayed graph issues nothing from the host.
        assert repeated == 0 if not on else repeated >= 4 * 4 and repeated % 4 == 0
    assert len(results[True]) == len(results[False]) == 9
    for i, (x, y) in enumerate(zip(results[True], results[False])):
        assert x.shape == y.shape and np.array_equal(x, y), f"step {i}: repeated layers differ from layers issued one by one"
    wq = {k: (plain.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()} if dtype == "bfloat16" else w
    assert_logits_close(results[True][0], plain.forward(wq, cfg, prompts[0][:150]), dtype, "a whole prompt through repeated layers")
    want_c = plain.forward(wq, cfg, prompts[2][:131])[130]
    assert_logits_close(results[True][4][0], want_c, dtype, "a portion through repeated layers")


def test_a_part_that_does_not_promise_to_launch_only_keeps_its_layers_out(tmp_path):
    """A toy feed-forward defined here (it adds its input with a torch operation) is registered and used in every
    layer: its layers run one by one, nothing is repeated, and the result is the one with replay switched off."""
    from tiny_inference_engine_b200 import StepEntry, StepRunner, load_model, make_cache
    from tiny_inference_engine_b200.ops import replay
    from tiny_inference_engine_b200.parts.feed_forward import SwiGLU
    from tiny_inference_engine_b200.parts.base import register_part

    class TorchSwiGLU(SwiGLU):
        launches_only = False

        def forward(self, h, ctx):
            out = super().forward(h, ctx)
            from tiny_inference_engine_b200.ops import SplitSum
            if isinstance(out, SplitSum):
                out = out.materialize(ctx.ws.rows("toy.out", out.M, out.N, self.dtype))
            out.add_(h)
            return out

    register_part("feed_forward", "swiglu", TorchSwiGLU, replace=True)
    try:
        cfg = dict(plain.TINY_D, num_hidden_layers=5)
        plain.write_model_dir(tmp_path, cfg, sharp_weights(cfg, 6))
        toks = np.random.default_rng(4).integers(0, cfg["vocab_size"], 40).tolist()
        got = []
        for on in (True, False):
            model = load_model(tmp_path, "bfloat16")
            model.layer_replay = on
            cache, states = make_cache(model, page_size=16, num_pages=8, max_requests=2)
            runner = StepRunner(model, cache, 64, 2, 64, states=states, use_graphs=False)
            req = cache.new_request()
            assert cache.reserve(req, 40)
            before = replay.layers_repeated
            runner.run([StepEntry(req, toks[:30], 0, [])])
            got.append(runner.run([StepEntry(req, toks[30:], 30, [9])]).float().cpu().numpy().copy())
            assert replay.layers_repeated == before
        assert np.array_equal(got[0], got[1])
    finally:
        register_part("feed_forward", "swiglu", SwiGLU, replace=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_engine_generates_the_same_tokens_with_repeated_layers(tmp_path, dtype):
    """Six layers alike under the scheduler: prompts cut into portions of 24 tokens beside decoding requests, a pool
    so small that requests are preempted and prefilled again, steps queued ahead, greedy and sampled requests. The
    tokens are those of the same engine with every layer issued from Python, and those of the plain implementation
    where it generates greedily in 32-bit."""
    from tiny_inference_engine_b200 import SamplingParams, ServingConfig, load_engine
    from tiny_inference_engine_b200.ops import replay
    cfg = dict(plain.TINY_D, num_hidden_layers=6)
    w = sharp_weights(cfg, 8)
    plain.write_model_dir(tmp_path, cfg, w)
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (5, 61, 30, 47, 2, 90)]
    params = [SamplingParams(max_tokens=6 + 3 * i, temperature=0.8 if i % 2 else 0.0, seed=70 + i) for i in range(6)]
    outs = {}
    for on in (True, False):
        eng = load_engine(tmp_path, dtype=dtype, num_pages=10, page_size=16, policy="fcfs", serving=ServingConfig(24, 8))
        eng.model.layer_replay = on
        before = replay.layers_repeated
        outs[on] = eng.generate_batch(prompts, params)
        while eng.has_work():
            eng.step()
        st = eng.stats()
        assert st.preemptions > 0 and st.steps_ahead > 0 and eng.cache.num_free() == 10
        assert (replay.layers_repeated > before) == on
    assert outs[True] == outs[False]
    if dtype == "float32":
        for i in (0, 2, 4):
            assert outs[True][i] == plain.generate(w, cfg, prompts[i], params[i].max_tokens)
