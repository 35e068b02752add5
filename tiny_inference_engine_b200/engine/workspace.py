"""Device buffers of a step, allocated once at their largest size and handed out by name.

Addresses are stable from the first use on, which is what a captured CUDA graph needs, and
steady-state stepping allocates nothing (the reference's arena: src/model/qwen3.cpp:109-146).
"""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, max_rows: int, device):
        self.max_rows = max_rows
        self.device = device
        self._rows: dict[tuple, torch.Tensor] = {}
        self._flat: dict[tuple, torch.Tensor] = {}

    def rows(self, name: str, n: int, width: int, dtype: torch.dtype) -> torch.Tensor:
        """[n, width] view of a buffer that holds max_rows rows."""
        key = (name, width, dtype)
        buf = self._rows.get(key)
        if buf is None:
            buf = torch.empty((self.max_rows, width), dtype=dtype, device=self.device)
            self._rows[key] = buf
        return buf[:n]

    def flat(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype)
        buf = self._flat.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(numel, dtype=dtype, device=self.device)
            self._flat[key] = buf
        return buf

    def zeros(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out (kernels that use it leave it zero)."""
        key = (name, dtype, "zeros")
        buf = self._flat.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.zeros(numel, dtype=dtype, device=self.device)
            self._flat[key] = buf
        return buf

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self._rows.values()) + list(self._flat.values()))
