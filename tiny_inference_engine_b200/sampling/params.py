"""Sampling parameters with the reference's names, defaults and checks (src/sampling/sampler.h:11-17,
src/sampling/sampler.cpp:10-16)."""
from __future__ import annotations

import math
from dataclasses import dataclass

from ..errors import InvalidArgument


@dataclass
class SamplingParams:
    temperature: float = 0.0   # 0 = greedy
    top_k: int = 0             # 0 = disabled
    top_p: float = 1.0         # 1 = disabled
    seed: int = 0
    max_tokens: int = 256      # generated tokens, including a final stop token

    def validate(self) -> None:
        if not (isinstance(self.temperature, (int, float)) and math.isfinite(self.temperature) and self.temperature >= 0):
            raise InvalidArgument(f"temperature must be finite and >= 0, got {self.temperature}")
        if not isinstance(self.top_k, int) or self.top_k < 0:
            raise InvalidArgument(f"top_k must be >= 0, got {self.top_k}")
        if not (isinstance(self.top_p, (int, float)) and 0.0 < self.top_p <= 1.0):
            raise InvalidArgument(f"top_p must be in (0, 1], got {self.top_p}")
        if not isinstance(self.seed, int) or self.seed < 0 or self.seed >= 2 ** 64:
            raise InvalidArgument(f"seed must be an unsigned 64-bit integer, got {self.seed}")
        if not isinstance(self.max_tokens, int) or self.max_tokens < 1:
            raise InvalidArgument(f"max_tokens must be >= 1, got {self.max_tokens}")

    @property
    def filters(self) -> bool:
        """Whether top-k or top-p narrows the candidates (with a temperature; greedy takes the first maximum
        whatever they say). Such rows run one more kernel after the plain draw. It depends on the request's
        parameters only, so its tokens never depend on what else is in a batch."""
        return self.temperature != 0.0 and (self.top_k > 0 or self.top_p < 1.0)

    def inv_temperature(self) -> float:
        """1/T as a float32 value; 0 stands for greedy (T == 0, or so small that 1/T is not finite)."""
        import numpy as np
        if self.temperature == 0.0:
            return 0.0
        with np.errstate(over="ignore", divide="ignore"):
            inv = np.float32(1.0) / np.float32(self.temperature)
        return float(inv) if np.isfinite(inv) else 0.0
