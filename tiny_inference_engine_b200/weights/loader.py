"""Weights by tensor name: where they come from, and the one check of names and shapes.

A `TensorSource` offers named tensors (a model folder's safetensors files, or random values).
`bind_check` compares what a model needs with what a source offers and raises ONE LoadError
that lists every missing tensor, every unexpected tensor and every wrong shape; the
reference stops at the first (src/model/qwen3.cpp:47-106), the rules are the same: exact
shapes, nothing left over, a tied model may carry a duplicate output table.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..errors import LoadError
from .safetensors import SafetensorsFile


@dataclass(frozen=True)
class TensorNeed:
    """What a part expects of one checkpoint tensor."""
    shape: tuple[int, ...]
    role: str = "matrix"      # "matrix" (N(0, std) when random), "norm" (1 + N(0, norm_std)), "table" (integers)
    optional: bool = False    # accepted when present, never required (a tied model's duplicate output table)


class TensorSource:
    def shapes(self) -> dict[str, tuple[tuple[int, ...], torch.dtype]]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype, on the CPU or already on the device."""
        raise NotImplementedError


class SafetensorsSource(TensorSource):
    """`model.safetensors`, or every shard named by `model.safetensors.index.json`'s weight_map
    (src/model/loader.cpp:224-249). A name in two shards is an error."""

    def __init__(self, model_dir):
        d = Path(model_dir)
        index = d / "model.safetensors.index.json"
        if index.exists():
            try:
                files = sorted(set(json.loads(index.read_text())["weight_map"].values()))
            except (OSError, KeyError, AttributeError, json.JSONDecodeError) as e:
                raise LoadError(f"{index}: {e}") from None
        else:
            files = ["model.safetensors"]
        self._where: dict[str, SafetensorsFile] = {}
        for name in files:
            f = SafetensorsFile(d / name)
            for tensor in f.entries:
                if tensor in self._where:
                    raise LoadError(f"duplicate tensor '{tensor}' ({self._where[tensor].path.name} and {name})")
                self._where[tensor] = f

    def shapes(self):
        from .safetensors import _DTYPES
        return {n: (f.entries[n].shape, _DTYPES[f.entries[n].dtype][2]) for n, f in self._where.items()}

    def get(self, name):
        return self._where[name].tensor(name)


class RandomSource(TensorSource):
    """Random values for exactly the tensors a model needs: matrices N(0, std), norm weights
    1 + N(0, norm_std), each tensor from its own generator seeded by (seed, ordinal of the
    name), so a tensor's values do not depend on which others exist."""

    def __init__(self, needs: dict[str, TensorNeed], seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                 norm_std: float = 0.01, device: str = "cpu"):
        self.needs = {n: t for n, t in needs.items() if not t.optional}
        self.seed, self.dtype, self.std, self.norm_std, self.device = seed, dtype, std, norm_std, device
        self._ordinal = {n: i for i, n in enumerate(sorted(self.needs))}

    def shapes(self):
        return {n: (t.shape, torch.float32 if t.role == "norm" else self.dtype) for n, t in self.needs.items()}

    def get(self, name):
        need = self.needs[name]
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1_000_003 + self._ordinal[name]) & 0x7FFFFFFFFFFFFFFF)
        if need.role == "norm":
            t = torch.randn(need.shape, generator=g, device=self.device, dtype=torch.float32)
            return t.mul_(self.norm_std).add_(1.0)
        if need.role == "table":
            return torch.zeros(need.shape, dtype=torch.int32, device=self.device)
        rows = need.shape[0]
        out = torch.empty(need.shape, dtype=self.dtype, device=self.device)
        step = max(1, (1 << 26) // max(1, out[0].numel()))  # bounded float32 scratch for large tables
        for r in range(0, rows, step):
            chunk = torch.randn(out[r:r + step].shape, generator=g, device=self.device, dtype=torch.float32)
            out[r:r + step] = chunk.mul_(self.std).to(self.dtype)
        return out


def bind_check(needs: dict[str, TensorNeed], source: TensorSource, what: str = "the model") -> None:
    have = source.shapes()
    missing = [n for n, t in needs.items() if not t.optional and n not in have]
    unexpected = [n for n in have if n not in needs]
    wrong = []
    for n, t in needs.items():
        if n in have:
            shape, dtype = have[n]
            if tuple(shape) != tuple(t.shape):
                wrong.append(f"'{n}' has shape {list(shape)}, expected {list(t.shape)}")
            elif t.role != "table" and dtype == torch.int32:
                wrong.append(f"'{n}' has dtype I32, expected a floating type")
    if missing or unexpected or wrong:
        parts = []
        if missing:
            parts.append("missing tensors: " + ", ".join(f"'{n}'" for n in missing))
        if unexpected:
            parts.append(f"tensors not used by {what}: " + ", ".join(f"'{n}'" for n in unexpected))
        if wrong:
            parts.append("wrong shapes: " + "; ".join(wrong))
        raise LoadError("checkpoint does not match " + what + ": " + " | ".join(parts))
