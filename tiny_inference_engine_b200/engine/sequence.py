"""A request's state in the engine (src/engine/sequence.h:12-30)."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from ..cache.manager import RequestCache
from ..sampling.params import SamplingParams


class SeqState(Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    FINISHED = "finished"


class FinishReason(Enum):
    NONE = "none"
    STOP = "stop"
    LENGTH = "length"
    ERROR = "error"
    CANCELLED = "cancelled"


@dataclass(eq=False)
class Sequence:
    id: int
    tokens: list[int]                 # prompt followed by generated tokens
    prompt_len: int
    params: SamplingParams
    cache: RequestCache | None = None
    num_computed: int = 0             # tokens whose keys and values are in the cache
    state: SeqState = SeqState.WAITING
    finish_reason: FinishReason = FinishReason.NONE
    waiting_since_step: int = 0       # scheduler step at which it last entered the waiting queue
    num_preemptions: int = 0

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def num_pending(self) -> int:
        return len(self.tokens) - self.num_computed
