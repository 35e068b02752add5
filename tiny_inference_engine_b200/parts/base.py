"""Registries and interfaces of the parts a layer is made of.

A part is built from a `PartSpec` (its kind and its sizes and constants) and the compute
dtype; it says which checkpoint tensors it needs, binds them, and runs on the rows of one
step. No part knows which model it is in. Kinds are registered by name, so a test or a
user can add a mixer, a feed-forward, a norm, a position encoding or a block arrangement
without touching this package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from ..config.spec import PartSpec
from ..errors import UnsupportedError
from ..weights.loader import TensorNeed


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer wants of the paged cache: keys and values of `kv_heads` x `head_dim` per
    token; kind "full" keeps every token, "window" only the last `window`."""
    kind: str
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps across steps (zero at position 0)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of every part."""

    # True for a part whose forward does its GPU work through this package's launchers only (no torch
    # operations), with arguments that depend on the step, on sizes and constants that layers built alike
    # share, and on tensors the part holds as attributes (its own, in a list or tuple, or in a part it holds the
    # same way; not in a dictionary). A run of layers made of such parts is issued by
    # one call after the first two (parts/layer_runs.py). Parts that do not say so run layer by layer.
    launches_only = False

    def needs(self) -> dict[str, TensorNeed]:
        """Checkpoint tensors by full name."""
        return {}

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        """Fetch the tensors named by needs(); `get(name)` returns them on the device in their stored dtype."""


class Norm(Part):
    def add_norm(self, x: torch.Tensor, delta, out: torch.Tensor, rows=None) -> None:
        """x (float32 residual stream) += delta when given; out = norm(x). With rows: only those rows, x untouched."""
        raise NotImplementedError

    def rows(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """Norm over the last axis of any 2-D view in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    def fused_table(self):
        """float32 inverse frequencies [rotary_dim / 2] if the encoding is a rotation the fused
        kernel can apply, else None (then `apply` is called on q and k)."""
        return None

    def apply(self, x: torch.Tensor, positions: torch.Tensor, heads: int, head_dim: int) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, h: torch.Tensor, ctx, cache, state) -> torch.Tensor:
        """h [T, D] in the compute dtype -> [T, D]. `cache` is a LayerCache (planes, group,
        whether this entry writes), or None; `state` is this entry's [slots, *shape] tensor or None."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """The arrangement of mixer, feed-forward and their norms in one layer."""

    def forward(self, x: torch.Tensor, pending, ctx, cache, state):
        """x: float32 residual stream [T, D]; pending: a delta not yet added to x (or None).
        Returns the new pending delta."""
        raise NotImplementedError


MIXERS: dict[str, Callable] = {}
FEED_FORWARDS: dict[str, Callable] = {}
NORMS: dict[str, Callable] = {}
POSITION_ENCODINGS: dict[str, Callable] = {}
BLOCKS: dict[str, Callable] = {}
_REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS,
               "block": BLOCKS}


def register_part(family: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """family: mixer | feed_forward | norm | position | block. factory(spec, dtype, prefix="") -> part."""
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise ValueError(f"{family} '{kind}' is already registered")
    reg[kind] = factory


def build_part(family: str, spec: PartSpec, dtype: torch.dtype, **kw):
    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise UnsupportedError(f"no {family} of kind '{spec.kind}' (registered: {', '.join(sorted(reg))})")
    return reg[spec.kind](spec, dtype, **kw)


def to_compute(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A matrix in the compute dtype: bfloat16 stays bfloat16 for serving; everything becomes
    float32 (exactly) for the 32-bit path; a 32-bit checkpoint served in bfloat16 is rounded once."""
    return t if t.dtype == dtype else t.to(dtype)
