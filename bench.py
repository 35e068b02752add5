#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, Qwen3-8B shape, random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload serving [--requests 64] [--kv-pages P]     (the Qwen3-4B serving mix; its own line)

One JSON line on stdout. `value` is decoded tokens per second at batch 8 with the timed steps
ending at the benchmark context (device time, CUDA events around K decode steps through the
step function); `e2e` is the same through the Python entry point (Engine.step: host token
ids in, sampled ids out, every step). `prefill` is one 2,048-token prompt in one step, timed first: a lone step
after a short idle against the burst peak (`ms`, `frac`) and steps in a row against the sustained peak
(`ms_back_to_back`, `frac_sustained`); `roofline` is the bytes a decode step has to read (every weight
it uses once, and the cache of the live requests) over its time, against the measured copy
bandwidth (`frac_b1`, `frac_b64`: the same for the two points); `points` holds decode at
batch 1 and 64, decode at batch 8 with contexts of 16,384 and 32,768 tokens (`frac_ctx...` beside them: there the
cache is the larger stream), the Qwen3-4B serving mix (`serving_4b`: the figures of `--workload serving`) and
the Qwen3-32B shape at batch 8 ending at context 8,192 (`decode_32b_b8_ctx8192`); `--no-extra` leaves the
last four out. Weights are 16 GB and the caches gigabytes, far more than the 126 MB L2, so no flush is
needed between steps.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# The Qwen3-8B shape: the headline configuration.
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
}
# The Qwen3-4B shape of the serving mix (`--workload serving`).
QWEN3_4B = dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True)
# A larger shape of the same architecture (`--shape 32b`): 64 layers, 64 query heads over 8 kv heads.
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64)
SHAPES = {"8b": ("Qwen3-8B", QWEN3_8B), "4b": ("Qwen3-4B", QWEN3_4B), "32b": ("Qwen3-32B", QWEN3_32B)}
FULL_LAYERS = 36
PAGE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        if os.environ.get('TIE_BENCH_NO_CLOCKS') == '1':
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([f.strip() for f in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def weight_bytes_per_decode_step(cfg, layers):
    D, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * D + D * q + 2 * I * D + D * I
    return 2 * (layers * per_layer + V * D)      # bfloat16; the embedding table is read one row per token


def kv_bytes_per_token(cfg, layers):
    return 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, T):
    D, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * D + D * q + 2 * I * D + D * I
    gemm = 2 * T * layers * per_layer + 2 * V * D            # one logits row
    attn = layers * 2 * 2 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) // 2   # causal QK^T and PV
    return gemm + attn


def serving_mix(args) -> dict:
    """The serving workload of the reference's own bench (bench/workload.cpp, bench/report.h:29-36) on the
    Qwen3-4B shape: `--requests` requests at once, prompt lengths uniform in [128, 4096] of uniform random ids,
    256 new tokens each at temperature 0.7, continuous batching with 512 tokens a step. One JSON line: generated
    tokens per second over the whole run, time to first token, time between tokens and request latency
    percentiles, mean sequences per step, preemptions."""
    import numpy as np
    import torch
    from tiny_inference_engine_b200 import (Engine, SamplingParams, Scheduler, SchedulerConfig, ServingConfig, StepRunner,
                                            load_model, make_cache)
    args.layers = args.layers or QWEN3_4B["num_hidden_layers"]
    cfg = dict(QWEN3_4B, num_hidden_layers=args.layers)
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "config.json").write_text(json.dumps(cfg))
        model = load_model(d, "bfloat16", random_weights=True, seed=0)
    n, new_tokens, budget = args.requests, 256, 512
    rng = np.random.default_rng(0)
    lengths = rng.integers(128, 4097, n)
    prompts = [rng.integers(0, cfg["vocab_size"], int(m)).tolist() for m in lengths]
    pages = int(sum((m + new_tokens) // PAGE + 2 for m in lengths)) if args.kv_pages <= 0 else args.kv_pages
    cache, states = make_cache(model, page_size=PAGE, num_pages=pages, max_requests=2 * n)
    serving = ServingConfig(max_tokens_per_step=budget, max_seqs=min(n, budget))
    runner = StepRunner(model, cache, budget, serving.max_seqs, serving.max_seqs, states=states)
    engine = Engine(model, cache, Scheduler(cache, SchedulerConfig(serving=serving)), serving, states=states, runner=runner)

    def run():
        stamps = {}
        engine.set_token_callback(lambda i, t: stamps.setdefault(i, []).append(time.perf_counter()))
        before = engine.stats()
        torch.cuda.synchronize()
        start = time.perf_counter()
        ids = [engine.add_request(p, SamplingParams(temperature=0.7, seed=k, max_tokens=new_tokens)) for k, p in enumerate(prompts)]
        while engine.has_work():
            engine.step()
        torch.cuda.synchronize()
        total = time.perf_counter() - start
        for i in ids:
            engine.release(i)
        return start, total, [stamps[i] for i in ids], before, engine.stats()

    run()                                                    # warm-up: kernels loaded, every decode graph captured
    start, total, stamps, st0, st1 = run()
    ttft = np.array([s[0] - start for s in stamps]) * 1e3
    itl = np.concatenate([np.diff(s) for s in stamps]) * 1e3
    e2e = np.array([s[-1] - start for s in stamps])
    generated = sum(len(s) for s in stamps)
    steps = st1.steps - st0.steps

    def pct(a):
        return {"p50": round(float(np.percentile(a, 50)), 2), "p90": round(float(np.percentile(a, 90)), 2),
                "p99": round(float(np.percentile(a, 99)), 2)}

    del engine, runner, cache, states, model
    torch.cuda.empty_cache()
    return {
        "metric": "generated tok/s, serving mix (Qwen3-4B bf16, 1 B200)", "value": round(generated / total, 1), "unit": "tokens/s",
        "requests": n, "prompt_tokens": int(lengths.sum()), "generated_tokens": generated, "seconds": round(total, 3),
        "total_tok_s": round((int(lengths.sum()) + generated) / total, 1), "ttft_ms": pct(ttft), "itl_ms": pct(itl), "e2e_s": pct(e2e),
        "steps": steps, "mean_seqs_per_step": round((st1.seqs_scheduled - st0.seqs_scheduled) / max(1, steps), 2),
        "preemptions": st1.preemptions - st0.preemptions, "steps_queued_ahead": st1.steps_ahead - st0.steps_ahead,
        "config": {"model": "Qwen3-4B shape", "layers": args.layers, "max_tokens_per_step": budget, "max_seqs": serving.max_seqs,
                   "kv_pages": pages, "page_size": PAGE, "temperature": 0.7, "new_tokens": new_tokens},
        "data": "synthetic (random weights N(0,0.02), uniform random token ids, all requests at time 0)"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096, help="context length at which the timed decode steps end")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the contract line is the default, 8b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (reported in config)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64 (and the extra points)")
    ap.add_argument("--no-extra", action="store_true", help="skip the long contexts, the serving mix and the 32B shape")
    ap.add_argument("--workload", default="decode", choices=["decode", "serving"],
                    help="decode: the contract line (default); serving: the Qwen3-4B serving mix, its own line")
    ap.add_argument("--requests", type=int, default=64, help="serving mix: concurrent requests")
    ap.add_argument("--kv-pages", type=int, default=0, help="serving mix: cache pages (0: enough for every request at once)")
    ap.add_argument("--profile", choices=["decode", "prefill", "mixed"], help="run two steps of one kind (mixed: 30 requests "
                    "decoding at context 2,048 beside a 482-token portion of a prompt, the serving default of 512 tokens a step), kernel by kernel, between "
                    "cudaProfilerStart/Stop (for ncu --profile-from-start off) and print no bench line")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a C++/Objective-C++ CMake project with a "
                          "Metal GPU backend (Apple only); pip cannot install it (no setup.py or pyproject.toml) and it has no CUDA path"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design (asked for --gpus {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "serving":
        print(json.dumps(serving_mix(args)))
        return 0

    import gc

    import numpy as np
    import torch
    from tiny_inference_engine_b200 import (Engine, SamplingParams, Scheduler, SchedulerConfig, ServingConfig, StepEntry,
                                            StepRunner, load_model, make_cache)
    from tiny_inference_engine_b200.ops import library as kernel_library

    pk, pk_src = peaks()
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    K, W, B, CTX = args.steps, args.warmup, args.batch, args.context
    rng = np.random.default_rng(0)
    clocks = ClockSampler()

    def build(config):
        with tempfile.TemporaryDirectory() as d:
            (Path(d) / "config.json").write_text(json.dumps(config))
            t0 = time.time()
            m = load_model(d, "bfloat16", random_weights=True, seed=0)
            torch.cuda.synchronize()
            print(f"[bench] model ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        return m

    model = build(cfg)
    V = cfg["vocab_size"]
    extra = not (args.no_points or args.no_extra or args.profile is not None)
    long_contexts = (16384, 32768) if extra else ()
    max_batch = B if args.no_points else max(B, 64)
    if args.profile == "mixed":
        max_batch = 32
    pages_per_seq = (CTX + PAGE - 1) // PAGE + 1
    num_pages = max([max_batch * pages_per_seq] + [B * (c // PAGE + 1) for c in long_contexts]) + 8
    cache, states = make_cache(model, page_size=PAGE, num_pages=num_pages, max_requests=max_batch * 2)
    chunk = max(args.prefill_tokens, 2048)
    runner = StepRunner(model, cache, max_tokens=chunk, max_seqs=max_batch, max_logit_rows=max_batch, states=states,
                        use_graphs=args.profile is None)

    def fill(run, pool, batch, length, reserve, random_fill=False):
        """`batch` requests with `length` tokens each in the cache: by real prefill in portions, or (the long contexts,
        where prefill would take longer than everything else together) by pages of random keys and values: what a
        decode step costs does not depend on what the keys are."""
        reqs = []
        if random_fill:
            for st in pool.storage:
                st.normal_(0.0, 1.0)
        for _ in range(batch):
            req = pool.new_request()
            assert pool.reserve(req, reserve)
            if not random_fill:
                toks = rng.integers(0, V, length)
                for at in range(0, length, chunk):
                    run.run([StepEntry(req, toks[at:at + chunk], at, [])])
            reqs.append(req)
        torch.cuda.synchronize()
        run.check()
        return reqs

    def decode_device(batch, steps, warmup, ctx=CTX, run=None, pool=None, random_fill=False):
        """Device time of `steps` decode steps of `batch` requests whose context ends at `ctx`."""
        run, pool = run or runner, pool or cache
        start = ctx - steps - warmup
        reqs = fill(run, pool, batch, start, ctx, random_fill)
        toks = rng.integers(0, V, (steps + warmup, batch))
        greedy = [(SamplingParams(), 0)] * batch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = replays0 = 0
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                launches0, replays0 = kernel_library.launch_count(), run.graph_replays
                e0.record()
            run.run([StepEntry(r, [int(toks[i, j])], start + i, [0]) for j, r in enumerate(reqs)], greedy)
        e1.record()
        torch.cuda.synchronize()
        run.check()
        ms = e0.elapsed_time(e1)
        per_graph = max(run.kernels_in_graph.values(), default=0)
        launches = (kernel_library.launch_count() - launches0) + (run.graph_replays - replays0) * per_graph
        for r in reqs:
            pool.release(r)
        return ms / steps, launches

    def hbm_frac(config, layers, batch, ctx, steps, ms):
        """Bytes a decode step has to read (weights once, the live requests' cache at the mean context of the
        timed steps) over its time, as a fraction of the copy bandwidth."""
        nbytes = weight_bytes_per_decode_step(config, layers) + batch * (ctx - steps / 2) * kv_bytes_per_token(config, layers)
        return round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    if args.profile is not None:
        greedy = [(SamplingParams(), 0)] * B
        if args.profile == "decode":
            reqs = fill(runner, cache, B, CTX - 4, CTX)
            steps = [[StepEntry(r, [int(rng.integers(0, V))], CTX - 4 + i, [0]) for r in reqs] for i in range(3)]
        elif args.profile == "mixed":
            reqs = fill(runner, cache, 30, 2048, CTX)
            prompt = fill(runner, cache, 1, 1024, CTX)[0]
            greedy = [(SamplingParams(), 0)] * 30
            steps = [[StepEntry(r, [int(rng.integers(0, V))], 2048 + i, [0]) for r in reqs] +
                     [StepEntry(prompt, rng.integers(0, V, 482), 1024 + 482 * i, [])] for i in range(3)]
        else:
            reqs = [cache.new_request() for _ in range(3)]
            for r in reqs:
                cache.reserve(r, args.prefill_tokens)
            steps = [[StepEntry(r, rng.integers(0, V, args.prefill_tokens), 0, [args.prefill_tokens - 1])] for r in reqs]
        runner.run(steps[0], greedy if args.profile != "prefill" else None)      # warm-up, not profiled
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for st in steps[1:]:
            runner.run(st, greedy if args.profile != "prefill" else None)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        runner.check()
        print(f"[bench] profiled two {args.profile} steps (batch {B}, context {CTX}, {args.layers} layers)", file=sys.stderr)
        return 0

    clocks.start()
    # prefill: one prompt, one step, the logits of its last token. Timed first, and in two ways. A lone step after the
    # GPU has idled for a fifth of a second is a burst of some 25 ms at full clocks: a kernel timed in isolation, which
    # is how the burst peak it is held against was measured (`ms`, `frac`). Steps one right after the other run under
    # the power cap like everything that goes on for long: those are held against the sustained peak
    # (`ms_back_to_back`, `frac_sustained`).
    T = args.prefill_tokens

    def prefill_once(idle_s):
        req = cache.new_request()
        cache.reserve(req, T)
        toks = rng.integers(0, V, T)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if idle_s:
            time.sleep(idle_s)
        e0.record()
        runner.run([StepEntry(req, toks, 0, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.release(req)
        return e0.elapsed_time(e1)

    for _ in range(3):                   # warm-up
        prefill_once(0.0)
    pre = sorted(prefill_once(0.2) for _ in range(5))[2]          # the median of five lone steps
    pre_b2b = sorted(prefill_once(0.0) for _ in range(5))[2]      # the median of five steps in a row
    runner.check()
    flops = prefill_flops(cfg, args.layers, T)

    ms_step, launches = decode_device(B, K, W)
    value = B / (ms_step / 1e3)

    points, point_fracs = {}, {}
    if not args.no_points:
        for b in (1, 64):
            steps_b = max(16, K // 4)
            ms_b, _ = decode_device(b, steps_b, W)
            points[f"decode_b{b}"] = round(b / (ms_b / 1e3), 1)
            point_fracs[f"frac_b{b}"] = hbm_frac(cfg, args.layers, b, CTX, steps_b, ms_b)
        for ctx in long_contexts:          # the cache is the larger stream here: decode attention sets the pace
            steps_c = 24
            ms_c, _ = decode_device(B, steps_c, W, ctx=ctx, random_fill=True)
            points[f"decode_b{B}_ctx{ctx}"] = round(B / (ms_c / 1e3), 1)
            point_fracs[f"frac_ctx{ctx}"] = hbm_frac(cfg, args.layers, B, ctx, steps_c, ms_c)

    # end to end through the Python entry point: host token ids in, sampled ids out, every step
    serving = ServingConfig(max_tokens_per_step=chunk, max_seqs=B)
    engine = Engine(model, cache, Scheduler(cache, SchedulerConfig(serving=serving, policy="fcfs")), serving, states=states,
                    runner=runner)
    # Prompts are prefilled one portion per step, so requests start decoding up to `stagger` steps apart;
    # every request still has tokens to generate until the last timed step and ends at the context CTX.
    stagger = B * ((CTX + chunk - 1) // chunk)
    start = CTX - K - W - stagger - 1
    for _ in range(B):
        engine.add_request(rng.integers(0, V, start).tolist(), SamplingParams(max_tokens=K + W + stagger + 1))
    while any(s.num_pending > 1 for s in engine.sequences.values()):
        engine.step()                       # prompts (not timed)
    for _ in range(W):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    steps_before = engine.stats().decode_tokens
    for _ in range(K - 1):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_tokens = engine.stats().decode_tokens - steps_before
    print(f"[bench] e2e: {K - 1} steps, {e2e_tokens} tokens, {e2e_s * 1e3 / (K - 1):.3f} ms per step, "
          f"{len(engine.scheduler.running)} running, {len(engine.scheduler.waiting)} waiting, "
          f"{engine.stats().preemptions} preemptions", file=sys.stderr, flush=True)
    h2d = runner.last_h2d_bytes          # the index arrays of a timed step: one copy from pinned memory
    while engine.has_work():
        engine.step()

    if extra:
        # the other two workloads, each with a model of its own: this one goes first
        del engine, runner, cache, states, model
        gc.collect()
        torch.cuda.empty_cache()
        mix = serving_mix(argparse.Namespace(layers=0, requests=64, kv_pages=0))
        points["serving_4b"] = {k: mix[k] for k in ("value", "total_tok_s", "ttft_ms", "itl_ms", "preemptions", "mean_seqs_per_step")}
        gc.collect()
        torch.cuda.empty_cache()
        big_name, big = SHAPES["32b"]
        big_model = build(big)
        b32, ctx32, steps32 = 8, 8192, 16
        big_cache, big_states = make_cache(big_model, page_size=PAGE, num_pages=b32 * (ctx32 // PAGE + 1) + 8, max_requests=2 * b32)
        big_runner = StepRunner(big_model, big_cache, max_tokens=64, max_seqs=b32, max_logit_rows=b32, states=big_states)
        ms32, _ = decode_device(b32, steps32, W, ctx=ctx32, run=big_runner, pool=big_cache, random_fill=True)
        points["decode_32b_b8_ctx8192"] = {"value": round(b32 / (ms32 / 1e3), 1), "ms_per_step": round(ms32, 3),
                                           "frac": hbm_frac(big, big["num_hidden_layers"], b32, ctx32, steps32, ms32)}
        del big_runner, big_cache, big_states, big_model
    clk = clocks.stop()

    step_bytes = weight_bytes_per_decode_step(cfg, args.layers) + B * (CTX - K / 2) * kv_bytes_per_token(cfg, args.layers)
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {B} ({shape_name} bf16, 1 B200)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "config": {"model": f"{shape_name} shape", "layers": args.layers, "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "global_batch": B, "seq_len": CTX,
                   "context_during_timed_steps": f"{CTX - K}..{CTX}", "page_size": PAGE, "parallelism": "single GPU", "order": "prefill timed first, then decode",
                   "l2": f"inputs larger than L2 ({weight_bytes_per_decode_step(cfg, args.layers) / 1e9:.0f} GB of weights per step)", "peaks": pk_src},
        "e2e": {"value": round(e2e_tokens / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": int(launches),
        "prefill": {"value": round(T / (pre / 1e3), 1), "tokens": T, "ms": round(pre, 3),
                    "frac": round(flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "timed": "median of five lone steps, each after 0.2 s of idle (a burst, like the peak)",
                    "ms_back_to_back": round(pre_b2b, 3),
                    "frac_sustained": round(flops / (pre_b2b / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), **point_fracs},
        "points": points,
        "clocks": clk,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
