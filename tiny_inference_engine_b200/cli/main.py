"""`tie generate -m DIR ...`: the reference's command (src/cli/args.cpp:70-158, src/cli/main.cpp:33-134) for a
model folder and token ids.

Options keep the reference's names, meanings and defaults where it has them: -m/--model, -p/--prompt,
--device, --max-tokens (256), --temp (0.7), --top-k (20), --top-p (0.8), --seed (0), --kv-mem (4G, with K/M/G
suffixes), and from its bench parser --max-seqs (64), --max-tokens-per-step (512), --policy
fcfs|srpt-aging, --aging (16). The reference's prompt is text; this engine has no tokenizer, so -p takes
token ids ("1 2 3" or "1,2,3"), or --prompt-len N draws N uniform ids from --seed. --device accepts
only cuda (the reference's metal|cpu do not exist here). The generated ids go to stdout, the reference's
statistics line to stderr. Exit codes: 1 for an engine error, 2 for anything else.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

USAGE = """usage: tie generate -m <model_dir> (-p "<ids>" | --prompt-len N) [options]
       tie make-random -o <model_dir> --config <config.json> [--seed S] [--dtype bfloat16|float32] [--device cpu|cuda]

generate options:
  -m, --model PATH      model directory (config.json + model.safetensors)
  -p, --prompt IDS      prompt token ids, separated by spaces or commas
  --prompt-len N        instead of -p: N uniform random token ids
  --random-weights      ignore model.safetensors; draw weights from --seed (needs only config.json)
  --device cuda         compute device (only cuda)
  --dtype D             bfloat16 (default) or float32
  --temp T              sampling temperature, 0 = greedy (default 0.7)
  --top-k K             keep the K most likely tokens, 0 = off (default 20)
  --top-p P             nucleus sampling threshold (default 0.8)
  --seed S              sampling seed (default 0)
  --max-tokens N        tokens to generate (default 256)
  --kv-mem SIZE         KV cache budget, e.g. 4G or 512M (default 4G)
  --page-size P         tokens per cache page (default 16)
  --max-seqs S          sequences per step (default 64)
  --max-tokens-per-step B  tokens per step (default 512)
  --policy fcfs|srpt-aging  admission order (default srpt-aging)
  --aging N             srpt-aging priority gained per step waited, in tokens (default 16)
  --stop-ids IDS        token ids that end generation
  --no-run-ahead        read every step's tokens before the next step is queued
"""


def parse_size(text: str) -> int:
    """A whole number with an optional K, M or G suffix (src/cli/args.cpp:105-126)."""
    from ..errors import InvalidArgument
    shift = {"K": 10, "M": 20, "G": 30}.get(text[-1:].upper(), 0)
    digits = text[:-1] if shift else text
    if not digits.isdigit():
        raise InvalidArgument(f"size '{text}' must be a whole number with an optional K, M or G suffix")
    value = int(digits) << shift
    if value == 0:
        raise InvalidArgument(f"size '{text}' must be positive")
    return value


def parse_ids(text: str) -> list[int]:
    from ..errors import InvalidArgument
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise InvalidArgument(f"token ids must be integers separated by spaces or commas, got '{text}'") from None


def run_generate(argv) -> int:
    from ..engine import ServingConfig, load_engine
    from ..engine.sequence import SeqState
    from ..errors import InvalidArgument
    from ..sampling import SamplingParams
    ap = argparse.ArgumentParser(prog="tie generate", add_help=False)
    ap.add_argument("-m", "--model")
    ap.add_argument("-p", "--prompt")
    ap.add_argument("--prompt-len", type=int)
    ap.add_argument("--random-weights", action="store_true")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--temp", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=20)
    ap.add_argument("--top-p", type=float, default=0.8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--kv-mem", default="4G")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-seqs", type=int, default=64)
    ap.add_argument("--max-tokens-per-step", type=int, default=512)
    ap.add_argument("--policy", default="srpt-aging")
    ap.add_argument("--aging", type=int, default=16)
    ap.add_argument("--stop-ids", default="")
    ap.add_argument("--no-run-ahead", action="store_true")
    try:
        o = ap.parse_args(argv)
    except SystemExit:
        raise InvalidArgument("bad command line; see `tie --help`") from None
    if not o.model:
        raise InvalidArgument("--model is required")
    if o.device != "cuda":
        raise InvalidArgument(f"--device must be cuda, got '{o.device}'")
    if (o.prompt is None) == (o.prompt_len is None):
        raise InvalidArgument("give exactly one of --prompt or --prompt-len")
    params = SamplingParams(temperature=o.temp, top_k=o.top_k, top_p=o.top_p, seed=o.seed, max_tokens=o.max_tokens)
    params.validate()

    t0 = time.perf_counter()
    engine = load_engine(o.model, dtype=o.dtype, kv_mem=parse_size(o.kv_mem), page_size=o.page_size,
                         serving=ServingConfig(o.max_tokens_per_step, o.max_seqs, run_ahead=not o.no_run_ahead), policy=o.policy, aging=o.aging,
                         stop_tokens=parse_ids(o.stop_ids), random_weights=o.random_weights, seed=o.seed)
    load_s = time.perf_counter() - t0
    if o.prompt is not None:
        prompt = parse_ids(o.prompt)
    else:
        import numpy as np
        prompt = np.random.default_rng(o.seed).integers(0, engine.model.spec.vocab_size, o.prompt_len).tolist()
    if not engine.stop_tokens:
        print("[tie] note: no stop ids given; generating until max_tokens", file=sys.stderr)

    times = []
    engine.set_token_callback(lambda seq_id, token: (times.append(time.perf_counter()), print(token, end=" ", flush=True)))
    start = time.perf_counter()
    seq_id = engine.add_request(prompt, params)
    try:
        while engine.sequence(seq_id).state != SeqState.FINISHED:
            engine.step()
    finally:
        print(flush=True)
    effective = engine.sequence(seq_id).params.max_tokens
    engine.release(seq_id)
    n = len(times)
    ttft = times[0] - start if n else 0.0
    prefill_rate = len(prompt) / ttft if ttft > 0 else 0.0
    decode_rate = (n - 1) / (times[-1] - times[0]) if n > 1 and times[-1] > times[0] else 0.0
    cache = engine.cache
    pages = -(-(len(prompt) + n) // cache.page_size)
    print(f"\n[tie] cuda | load {load_s:.2f} s | prompt {len(prompt)} tok | ttft {ttft * 1e3:.0f} ms | prefill "
          f"{prefill_rate:.1f} tok/s | decode {decode_rate:.1f} tok/s | {n} tok generated | kv {pages} blocks for "
          f"{len(prompt) + n} tok, pool {cache.num_pages} blocks ({cache.bytes_per_page * cache.num_pages / 2 ** 30:.2f} GiB)",
          file=sys.stderr)
    if effective < o.max_tokens:
        print(f"[tie] note: max_tokens clamped to {effective} by the KV cache / context", file=sys.stderr)
    return 0


def run_make_random(argv) -> int:
    from ..engine.loading import parse_dtype
    from ..errors import InvalidArgument
    from ..weights import write_random_model
    ap = argparse.ArgumentParser(prog="tie make-random", add_help=False)
    ap.add_argument("-o", "--out")
    ap.add_argument("--config")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--device", default="cpu")
    try:
        o = ap.parse_args(argv)
    except SystemExit:
        raise InvalidArgument("bad command line; see `tie --help`") from None
    if not o.out or not o.config:
        raise InvalidArgument("--out and --config are required")
    with open(o.config) as f:
        cfg = json.load(f)
    d = write_random_model(o.out, cfg, o.seed, parse_dtype(o.dtype), device=o.device)
    print(f"[tie] wrote {d}/config.json and {d}/model.safetensors", file=sys.stderr)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        (sys.stdout if argv else sys.stderr).write(USAGE)
        return 0 if argv else 1
    from ..errors import InvalidArgument, TieError
    try:
        if argv[0] == "generate":
            return run_generate(argv[1:])
        if argv[0] == "make-random":
            return run_make_random(argv[1:])
        raise InvalidArgument(f"unknown command '{argv[0]}'")
    except TieError as e:
        print(f"tie: error: {e}", file=sys.stderr)
        return 1
    except Exception as e:  # noqa: BLE001
        print(f"tie: internal error: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
