"""Device buffers of a step, handed out by name.

Row buffers are allocated once at their largest size. A flat buffer grows when a step asks for more
than any step before it; the smaller buffer it replaces is kept, never given back, because a
captured CUDA graph may still write to its address (and read from it in the same graph). Callers
that know their largest need say so (`capacity`), so that growth is the exception. Steady-state
stepping allocates nothing (the reference's arena: src/model/qwen3.cpp:109-146).
"""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, max_rows: int, device):
        self.max_rows = max_rows
        self.device = device
        self._rows: dict[tuple, torch.Tensor] = {}
        self._flat: dict[tuple, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []      # outgrown buffers: captured graphs may still use them

    def rows(self, name: str, n: int, width: int, dtype: torch.dtype) -> torch.Tensor:
        """[n, width] view of a buffer that holds max_rows rows."""
        if n > self.max_rows:
            raise ValueError(f"workspace '{name}': {n} rows asked of a workspace of {self.max_rows}")
        key = (name, width, dtype)
        buf = self._rows.get(key)
        if buf is None:
            buf = torch.empty((self.max_rows, width), dtype=dtype, device=self.device)
            self._rows[key] = buf
        return buf[:n]

    def flat(self, name: str, numel: int, dtype: torch.dtype, capacity: int = 0) -> torch.Tensor:
        """At least `numel` elements; allocated with max(numel, capacity) the first time."""
        return self._grow((name, dtype), numel, capacity, lambda n: torch.empty(n, dtype=dtype, device=self.device))

    def _grow(self, key, numel: int, capacity: int, make) -> torch.Tensor:
        buf = self._flat.get(key)
        if buf is None or buf.numel() < numel:
            if buf is not None:
                self._retired.append(buf)
            buf = make(max(numel, capacity, 2 * buf.numel() if buf is not None else 0))
            self._flat[key] = buf
        return buf

    def zeros(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out (kernels that use it leave it zero)."""
        return self._grow((name, dtype, "zeros"), numel, 0, lambda n: torch.zeros(n, dtype=dtype, device=self.device))

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in list(self._rows.values()) + list(self._flat.values()) + self._retired)
