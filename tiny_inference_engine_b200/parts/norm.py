"""RMSNorm: (x * 1/sqrt(mean(x^2) + eps)) * w, sums and scale in float32
(src/backend/cpu/cpu_backend.cpp:141-159). The weight is kept in float32 whatever the
checkpoint stores (src/model/qwen3.cpp:60-71)."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorNeed
from .base import Norm, register_part


class RMSNorm(Norm):
    launches_only = True
    takes_split_sum = True      # add_norm adds the partial sums of a split product itself
    fusable_rms = True          # exactly the formula above, with `weight` (float32) and `eps`

    def __init__(self, spec, dtype, prefix: str = ""):
        self.name = prefix + spec["name"]
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.dtype = dtype
        self.weight = None

    def needs(self):
        return {self.name: TensorNeed((self.size,), "norm")}

    def bind(self, get):
        self.weight = get(self.name).to(torch.float32).contiguous()

    def add_norm(self, x, delta, out, rows=None):
        ops.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)

    def rows(self, x, out):
        ops.rmsnorm_rows(x, self.weight, self.eps, out)


register_part("norm", "rmsnorm", RMSNorm, replace=True)
