"""From a model folder to a running engine: the calls a user makes."""
from __future__ import annotations

from pathlib import Path

import torch

from ..cache.manager import CacheManager
from ..cache.state_slots import StateSlots
from ..config.registry import load_config
from ..errors import InvalidArgument
from ..parts.model import Model
from ..weights.loader import RandomSource, SafetensorsSource
from .engine import Engine
from .scheduler import Scheduler, SchedulerConfig, ServingConfig
from .step import StepRunner

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return DTYPES[str(name)]
    except KeyError:
        raise InvalidArgument(f"dtype must be bfloat16 or float32, got '{name}'") from None


def load_model(model_dir, dtype="bfloat16", device="cuda", random_weights: bool = False, seed: int = 0) -> Model:
    """The model class is chosen by config.json. With random_weights the folder needs only
    config.json: weights are drawn on the device (matrices N(0, 0.02), norms 1 + N(0, 0.01))."""
    dt = parse_dtype(dtype)
    arch, cfg, spec = load_config(model_dir)
    model = Model(spec, dt)
    model.config = cfg
    if random_weights:
        source = RandomSource(model.needs(), seed, dtype=dt, device=device)
    else:
        source = SafetensorsSource(Path(model_dir))
    return model.load(source, device=device)


def make_cache(model: Model, page_size: int = 16, num_pages: int | None = None, kv_mem: int | None = None,
               max_requests: int = 64, device="cuda", window_requests: int | None = None,
               window_step_tokens: int = 0) -> tuple[CacheManager, StateSlots]:
    """The cache and the state slots of a model. `max_requests` is how many requests can hold state of fixed
    size at once; with `window_requests` layers that keep a window of keys get pages for that many requests
    only (`CacheManager`), the rest of the budget goes to the layers that keep every key."""
    states = StateSlots(model.state_needs(), max_requests, device=device)
    cache = CacheManager(model.cache_needs(), page_size, num_pages=num_pages, budget_bytes=kv_mem, dtype=model.dtype,
                         device=device, state_slots=states, window_requests=window_requests,
                         window_step_tokens=window_step_tokens)
    return cache, states


def load_engine(model_dir, dtype="bfloat16", kv_mem: int = 4 << 30, page_size: int = 16, num_pages: int | None = None,
                serving: ServingConfig | None = None, policy: str = "srpt-aging", aging: int = 16,
                stop_tokens=(), random_weights: bool = False, seed: int = 0, device="cuda",
                watermark_pages: int = -1) -> Engine:
    """Model folder -> Engine, wired the way the reference's CLI wires its own (src/cli/main.cpp:33-69)."""
    serving = serving or ServingConfig()
    serving.validate()
    model = load_model(model_dir, dtype, device, random_weights, seed)
    # Requests that hold pages or a state slot at one time: those running, and those whose last token is still
    # on its way from the GPU when the step behind it was already decided (they have left the scheduler).
    holders = 2 * serving.max_seqs
    cache, states = make_cache(model, page_size, num_pages, None if num_pages else kv_mem, max_requests=holders,
                               device=device, window_requests=holders, window_step_tokens=serving.max_tokens_per_step)
    scheduler = Scheduler(cache, SchedulerConfig(serving=serving, policy=policy, aging=aging,
                                                 watermark_pages=watermark_pages))
    runner = StepRunner(model, cache, serving.max_tokens_per_step, serving.max_seqs, serving.max_seqs, states=states,
                        device=device)
    return Engine(model, cache, scheduler, serving, stop_tokens=stop_tokens, states=states, runner=runner)
