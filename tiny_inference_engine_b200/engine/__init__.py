"""Step function, scheduler and engine."""
from .engine import Engine, EngineStats
from .loading import load_engine, load_model, make_cache, parse_dtype
from .scheduler import POLICIES, ScheduledBatch, Scheduler, SchedulerConfig, ServingConfig
from .sequence import FinishReason, SeqState, Sequence
from .step import StepContext, StepEntry, StepRunner
from .workspace import Workspace

__all__ = ["Engine", "EngineStats", "load_engine", "load_model", "make_cache", "parse_dtype", "POLICIES",
           "ScheduledBatch", "Scheduler", "SchedulerConfig", "ServingConfig", "FinishReason", "SeqState", "Sequence",
           "StepContext", "StepEntry", "StepRunner", "Workspace"]
