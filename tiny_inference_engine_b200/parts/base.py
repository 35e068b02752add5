"""Registries and interfaces of the parts a layer is made of.

A part is built from a `PartSpec` (its kind and its sizes and constants) and the compute
dtype; it says which checkpoint tensors it needs, binds them, and runs on the rows of one
step. No part knows which model it is in. Kinds are registered by name, so a test or a
user can add a mixer, a feed-forward, a norm, a position encoding, a block arrangement, a
token embedding or an output head without touching this package.
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
    # True only for a norm that computes out = (x / sqrt(mean(x^2) + eps)) * weight with a float32 `weight`
    # and an `eps` of its own: kernels that fuse that formula into other work (the q/k norm with the rotation
    # and the cache append) may then stand in for `rows`. Any other formula leaves it False and is called.
    fusable_rms = False

    def add_norm(self, x: torch.Tensor, delta, out: torch.Tensor, rows=None) -> None:
        """x (float32 residual stream) += delta when given; out = norm(x). With rows: only those rows, x untouched."""
        raise NotImplementedError

    def rows(self, x: torch.Tensor, out: torch.Tensor) -> None:
        """Norm over the last axis of any 2-D view in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    # True for an encoding that leaves q and k as they are: the mixer then need not call it at all.
    is_identity = False

    def fused_table(self):
        """float32 inverse frequencies [rotary_dim / 2] if the encoding is a rotation the fused
        kernel can apply, else None (then `apply` is called on q and k)."""
        return None

    def score_scale(self) -> float:
        """A factor on the attention scores that the encoding asks for (a rotation stretched to longer
        contexts may come with one); the mixer multiplies its softmax scale by it."""
        return 1.0

    def apply(self, x: torch.Tensor, positions: torch.Tensor, heads: int, head_dim: int) -> None:
        raise NotImplementedError


class Mixer(Part):
    # For a mixer that keeps state (`state_need`): True if its forward reads the step through the device tensors of
    # `ctx` only (never `ctx.host`) and copes with the sequences that pad a captured batch (state slot -1, no keys):
    # decode steps of a model with such mixers are then captured as CUDA graphs like those of a model without state.
    # False (the default) keeps every step of the model out of graphs.
    graph_safe = False

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


class Embedding(Part):
    """Token ids to the float32 residual stream."""

    def forward(self, tokens: torch.Tensor, x: torch.Tensor) -> None:
        """tokens int32 [T] -> x float32 [T, D] (written in place)."""
        raise NotImplementedError


class OutputHead(Part):
    """The rows that reached the final norm to float32 logits. Built with `embedding=` the model's embedding
    part, for heads that share its table."""

    def forward(self, last: torch.Tensor, logits: torch.Tensor) -> None:
        """last [R, D] in the compute dtype -> logits float32 [R, V] (written in place)."""
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
EMBEDDINGS: dict[str, Callable] = {}
HEADS: dict[str, Callable] = {}
_REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS,
               "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS}


def register_part(family: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """family: mixer | feed_forward | norm | position | block | embedding | head.
    factory(spec, dtype, prefix="") -> part; a block's factory takes (layer_spec, dtype), a head's
    (spec, dtype, embedding=the model's embedding part)."""
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
