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
               max_requests: int = 64, device="cuda") -> tuple[CacheManager, StateSlots]:
    states = StateSlots(model.state_needs(), max_requests, device=device)
    cache = CacheManager(model.cache_needs(), page_size, num_pages=num_pages, budget_bytes=kv_mem, dtype=model.dtype,
                         device=device, state_slots=states)
    return cache, states


def load_engine(model_dir, dtype="bfloat16", kv_mem: int = 4 << 30, page_size: int = 16, num_pages: int | None = None,
                serving: ServingConfig | None = None, policy: str = "srpt-aging", aging: int = 16,
                stop_tokens=(), random_weights: bool = False, seed: int = 0, device="cuda") -> Engine:
    """Model folder -> Engine, wired the way the reference's CLI wires its own (src/cli/main.cpp:33-69)."""
    serving = serving or ServingConfig()
    serving.validate()
    model = load_model(model_dir, dtype, device, random_weights, seed)
    cache, states = make_cache(model, page_size, num_pages, None if num_pages else kv_mem,
                               max_requests=serving.max_seqs * 4, device=device)
    scheduler = Scheduler(cache, SchedulerConfig(serving=serving, policy=policy, aging=aging))
    runner = StepRunner(model, cache, serving.max_tokens_per_step, serving.max_seqs, serving.max_seqs, states=states,
                        device=device)
    return Engine(model, cache, scheduler, serving, stop_tokens=stop_tokens, states=states, runner=runner)
