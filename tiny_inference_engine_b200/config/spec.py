"""The description of a model as data: which parts make up each layer and in which order the layers run.

An architecture turns its typed configuration into a `ModelSpec`. Everything below the
registry (weights binding, parts, cache manager, step function) reads only the spec, so a
part never knows which model it is in, and a new architecture is a new function that
returns a spec.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """One part: its kind (a key of the parts registry) and its sizes and constants."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a sequence mixer and a feed-forward, each behind its own norm, arranged by `block`.

    `prefix` is the checkpoint name prefix of the layer (for instance "model.layers.3.").
    """
    prefix: str
    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One position of the run order. `layer` indexes `ModelSpec.layers`; a layer may be named by
    several entries. `cache_of` names an EARLIER entry whose cache this entry reads instead
    of writing its own (its mixer then computes no keys and values)."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec          # params: name (checkpoint tensor)
    layers: tuple[LayerSpec, ...]
    run_order: tuple[RunEntry, ...]
    final_norm: PartSpec         # params: name, eps
    head: PartSpec               # params: name, tied (bool)

    def validate(self) -> None:
        from ..errors import InvalidArgument
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise InvalidArgument(f"run order entry {i} names layer {e.layer}; the model has {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise InvalidArgument(f"run order entry {i} reads the cache of entry {e.cache_of}, which is not earlier")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise InvalidArgument(f"run order entry {i} reads the cache of entry {e.cache_of}, which has none of its own")
