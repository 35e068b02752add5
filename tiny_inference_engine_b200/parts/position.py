"""Rotary position encoding, rotate-half over the first `rotary_dim` dims of a head:
inv_freq[i] = 1 / theta^(2i / rotary_dim) in float32, angle = float(pos) * inv_freq[i]
(src/backend/rope.h:9-13, src/backend/cpu/cpu_backend.cpp:161-193). The table is computed
once on the host, as the reference does, so that angles are the same float32 products."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..errors import InvalidArgument
from .base import PositionEncoding, register_part


class RotaryEncoding(PositionEncoding):
    launches_only = True

    def __init__(self, spec, dtype, prefix: str = ""):
        self.theta = float(spec["theta"])
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise InvalidArgument(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        i = np.arange(self.rotary_dim // 2, dtype=np.float32)
        expo = (np.float32(2.0) * i) / np.float32(self.rotary_dim)
        self.inv_freq_host = (np.float32(1.0) / np.power(np.float32(self.theta), expo, dtype=np.float32)).astype(np.float32)
        self._table = None

    def fused_table(self):
        if self._table is None:
            self._table = torch.from_numpy(self.inv_freq_host).cuda()
        return self._table

    def apply(self, x, positions, heads, head_dim):
        ops.rope(x, positions, self.fused_table(), heads, head_dim)


class NoPositionEncoding(PositionEncoding):
    """Leaves q and k as they are."""

    launches_only = True
    is_identity = True

    def __init__(self, spec=None, dtype=None, prefix: str = ""):
        pass

    def apply(self, x, positions, heads, head_dim):
        return None


register_part("position", "rope", RotaryEncoding, replace=True)
register_part("position", "none", NoPositionEncoding, replace=True)
