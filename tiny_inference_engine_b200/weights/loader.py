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
    1 + N(0, norm_std). Element i of a tensor is a function of (seed, ordinal of the tensor's name among
    the sorted names, i) alone (weights/counter_random.py): the same bits whether drawn on the CPU or on
    the GPU, in one piece or in several, so that a random model can be named by its configuration and its
    seed across tools (`--random-weights`, `tie make-random`, bench.py)."""

    def __init__(self, needs: dict[str, TensorNeed], seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                 norm_std: float = 0.01, device: str = "cpu"):
        self.needs = {n: t for n, t in needs.items() if not t.optional}
        self.seed, self.dtype, self.std, self.norm_std, self.device = seed, dtype, std, norm_std, device
        self._ordinal = {n: i for i, n in enumerate(sorted(self.needs))}

    def shapes(self):
        return {n: (t.shape, torch.float32 if t.role == "norm" else self.dtype) for n, t in self.needs.items()}

    def get(self, name):
        from .counter_random import standard_normal
        need = self.needs[name]
        ordinal = self._ordinal[name]
        if need.role == "table":
            return torch.zeros(need.shape, dtype=torch.int32, device=self.device)
        numel = 1
        for n in need.shape:
            numel *= n
        if need.role == "norm":
            z = standard_normal(self.seed, ordinal, 0, numel, self.device)
            return (z * self.norm_std + 1.0).to(torch.float32).reshape(need.shape)
        out = torch.empty(numel, dtype=self.dtype, device=self.device)
        step = 1 << 24                              # bounded float64 scratch for large tables
        for at in range(0, numel, step):
            n = min(step, numel - at)
            out[at:at + n] = (standard_normal(self.seed, ordinal, at, n, self.device) * self.std).to(torch.float32).to(self.dtype)
        return out.reshape(need.shape)


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
