"""A model built from a `ModelSpec`: embedding, the layers in their run order, final norm, output table."""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from ..config.spec import ModelSpec
from ..errors import InvalidArgument, UnsupportedError
from ..ops import replay as layer_replay
from ..weights.loader import TensorNeed, TensorSource, bind_check
from .base import BLOCKS, CacheNeed, StateNeed, build_part
from .layer_runs import LayerRuns, same_handoff


@dataclass
class LayerCache:
    """What a run entry sees of the cache: its planes, its group, and whether it writes them."""
    k: torch.Tensor | None
    v: torch.Tensor | None
    group: int
    writes: bool


def _build_block(layer_spec, dtype):
    kind = layer_spec.block.kind
    if kind not in BLOCKS:
        raise UnsupportedError(f"no block of kind '{kind}' (registered: {', '.join(sorted(BLOCKS))})")
    return BLOCKS[kind](layer_spec, dtype)


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise InvalidArgument(f"compute dtype must be float32 or bfloat16, got {dtype}")
        spec.validate()
        self.spec, self.dtype = spec, dtype
        self.embedding = build_part("embedding", spec.embedding, dtype)
        self.layers = [_build_block(l, dtype) for l in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype)
        self.head = build_part("head", spec.head, dtype, embedding=self.embedding)
        self.loaded = False
        # Layers built alike are issued by one call after the first two of their run (ops/replay.py);
        # TIE_NO_LAYER_REPLAY=1 issues every layer from Python.
        self.layer_replay = os.environ.get("TIE_NO_LAYER_REPLAY") != "1"
        self._forwards = 0
        self._layer_runs: dict[int, LayerRuns] = {}     # id(cache) -> runs (checked against the cache itself)

    # -- what the model needs of a checkpoint, of the cache and of per-request state
    def needs(self) -> dict[str, TensorNeed]:
        n = dict(self.embedding.needs())
        for l in self.layers:
            n.update(l.needs())
        n.update(self.final_norm.needs())
        n.update(self.head.needs())
        return n

    def cache_needs(self) -> list[CacheNeed | None]:
        """Per run entry: the cache it owns (None if it has none or reads another entry's)."""
        return [self.layers[e.layer].mixer.cache_need() if e.cache_of is None else None for e in self.spec.run_order]

    def state_needs(self) -> list[StateNeed | None]:
        return [self.layers[e.layer].mixer.state_need() for e in self.spec.run_order]

    def load(self, source: TensorSource, device="cuda") -> "Model":
        needs = self.needs()
        bind_check(needs, source, what=self.spec.architecture)

        def get(name: str) -> torch.Tensor:
            return source.get(name).to(device, non_blocking=False)

        self.embedding.bind(get)
        for l in self.layers:
            l.bind(get)
        self.final_norm.bind(get)
        self.head.bind(get)
        self.loaded = True
        self._forwards = 0
        self._layer_runs.clear()
        return self

    def _runs_for(self, ctx, cache, states) -> "LayerRuns | None":
        """The runs of alike layers for this cache, or None when layers are to be issued one by one: replay
        switched off, a per-layer hook, or the model's first forward (tensors that parts make at first use
        exist only after it)."""
        if not self.layer_replay or ctx.layer_hook is not None or self._forwards == 0:
            return None
        runs = self._layer_runs.get(id(cache))
        if runs is None or (runs.cache_ref() if runs.cache_ref is not None else None) is not cache or not runs.alive():
            if len(self._layer_runs) > 8:
                self._layer_runs.clear()
            runs = self._layer_runs[id(cache)] = LayerRuns(self, cache, states)
        return runs if runs.run_end else None

    # -- one step over the rows of ctx; returns float32 logits [R, V] or None when no row is wanted
    def forward(self, ctx, cache, states) -> torch.Tensor | None:
        T, D = ctx.T, self.spec.hidden_size
        ctx.ws_dtype = self.dtype
        x = ctx.ws.rows("model.x", T, D, torch.float32)
        self.embedding.forward(ctx.tokens, x)
        pending = None
        order = self.spec.run_order

        def run_entry(i, pending):
            entry = order[i]
            owner = i if entry.cache_of is None else entry.cache_of
            view = cache.layer_cache(owner, writes=entry.cache_of is None) if cache is not None else None
            state = states.tensor(i) if states is not None else None
            pending = self.layers[entry.layer].forward(x, pending, ctx, view, state)
            if ctx.layer_hook is not None:
                ctx.layer_hook(i, x, pending)
            return pending

        runs = self._runs_for(ctx, cache, states)
        i = 0
        while i < len(order):
            end = runs.run_end.get(i) if runs is not None else None
            pending = run_entry(i, pending)
            i += 1
            if end is None:
                continue
            # Entries i-1 .. end are built alike. The first may have been handed something else than it hands
            # on (nothing, at the start of the model), so the second one is recorded; if it hands on what it
            # was handed, the rest of the run makes the same calls with its own tensors' addresses.
            handed = pending
            with layer_replay.record() as calls:
                pending = run_entry(i, pending)
            i += 1
            spans = runs.spans(i - 1, i - 2) if same_handoff(handed, pending) else None
            plan = None
            if spans is not None:
                key = (i - 2, tuple(calls))
                plan = runs.plans.get(key)
                if plan is None:
                    if len(runs.plans) >= 64:
                        runs.plans.clear()
                    plan = runs.plans[key] = layer_replay.plan(calls, spans)
            if plan is not None:
                layer_replay.run(plan, runs.table[i - 2][2:])
                i = end + 1
        self._forwards += 1
        if ctx.R == 0:
            return None
        last = ctx.logit_ws.rows("model.last", ctx.R, D, self.dtype)
        from .block import as_delta
        self.final_norm.add_norm(x, as_delta(pending, self.final_norm, ctx, "block.delta"), last, rows=ctx.logit_rows)
        logits = ctx.logit_ws.rows("model.logits", ctx.R, self.spec.vocab_size, torch.float32)
        self.head.forward(last, logits)
        return logits


def expected_tensors(spec: ModelSpec) -> dict[str, TensorNeed]:
    """Names, shapes and roles of the checkpoint tensors of a model description (no device needed)."""
    return Model(spec, torch.bfloat16).needs()
