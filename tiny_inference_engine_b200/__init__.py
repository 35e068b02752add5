"""A small, whole LLM inference engine for one NVIDIA B200 and the Qwen3 dense architecture.

    from tiny_inference_engine_b200 import load_engine, SamplingParams
    engine = load_engine("/path/to/model", dtype="bfloat16", kv_mem=4 << 30)
    ids = engine.generate([1, 2, 3], SamplingParams(temperature=0.7, seed=1, max_tokens=32))
"""
from .errors import CapacityError, InvalidArgument, LoadError, TieError, UnsupportedError
from .config import Qwen3Config, load_config, register_architecture
from .engine import (Engine, EngineStats, ServingConfig, SchedulerConfig, Scheduler, StepEntry, StepRunner,
                     load_engine, load_model, make_cache)
from .sampling import SamplingParams
from .weights import write_random_model

__all__ = ["CapacityError", "InvalidArgument", "LoadError", "TieError", "UnsupportedError", "Qwen3Config",
           "load_config", "register_architecture", "Engine", "EngineStats", "ServingConfig", "SchedulerConfig",
           "Scheduler", "StepEntry", "StepRunner", "load_engine", "load_model", "make_cache", "SamplingParams",
           "write_random_model"]
__version__ = "0.1.0"
