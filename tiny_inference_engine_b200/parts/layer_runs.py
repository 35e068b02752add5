"""Runs of layers that are built alike, so that a step can issue them with one call (ops/replay.py).

Two run entries are alike when their layers are of the same classes with the same sizes and constants, hold
tensors of the same shapes, use the same cache group in the same way, keep no state of their own, and every
part in them says `launches_only`. Such layers make the same launcher calls with the same arguments except
for the addresses of their own tensors and cache planes, which `LayerRuns` lists per entry in a fixed order.
"""
from __future__ import annotations

import weakref

import numpy as np
import torch

from ..ops import replay as layer_replay
from .base import Part

_PACKAGE = __name__.split(".")[0]


def walk_part(obj, tensors: list, scalars: list, seen: set) -> bool:
    """Collects, in attribute order, the tensors `obj` and the parts inside it hold, and the sizes and constants
    beside them (names of checkpoint tensors and addresses left out). Layers built alike give lists that differ in
    the tensors' addresses only. Returns whether every part met says `launches_only`."""
    ok = bool(getattr(obj, "launches_only", False)) if isinstance(obj, Part) else True
    seen.add(id(obj))
    for name, v in vars(obj).items():
        for item in (v if isinstance(v, (list, tuple)) else (v,)):
            if isinstance(item, torch.Tensor):
                tensors.append(item)
            elif isinstance(item, (bool, float, torch.dtype)) or item is None:
                scalars.append((name, item))
            elif isinstance(item, int):
                if item < (1 << 32) and not name.endswith("_ptr"):
                    scalars.append((name, item))
            elif isinstance(item, dict):
                if any(isinstance(x, (torch.Tensor, Part)) for x in item.values()):
                    ok = False      # tensors in a dictionary have no fixed order to list them in
            elif isinstance(item, (str, np.ndarray)):
                continue
            elif hasattr(item, "__dict__") and id(item) not in seen and (
                    isinstance(item, Part) or type(item).__module__.split(".")[0] == _PACKAGE):
                scalars.append((name, type(item).__qualname__))
                ok = walk_part(item, tensors, scalars, seen) and ok
            elif hasattr(item, "__dict__") and id(item) not in seen:
                ok = False      # an object of unknown kind: what it holds cannot be listed
    return ok


def _extent_bytes(t: torch.Tensor) -> int:
    if t.numel() == 0:
        return 0
    return (sum((n - 1) * st for n, st in zip(t.shape, t.stride())) + 1) * t.element_size()


def same_handoff(a, b) -> bool:
    """Whether two layers handed on their pending delta in the same form at the same place."""
    from ..ops import SplitSum
    if isinstance(a, SplitSum) and isinstance(b, SplitSum):
        return (a.partial.data_ptr(), a.splits, a.M, a.N) == (b.partial.data_ptr(), b.splits, b.M, b.N)
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
        return (a.data_ptr(), a.shape, a.stride(), a.dtype) == (b.data_ptr(), b.shape, b.stride(), b.dtype)
    return False


class LayerRuns:
    """Runs of consecutive run entries whose layers are built alike, for one model and one cache: which entries
    start a run and where it ends, and per entry the addresses of its tensors and cache planes in slot order.
    A run has at least `MIN_RUN` entries: looking the recorded layer's tensors up and turning its calls into
    a list costs about as much host time as issuing two layers from Python."""

    MIN_RUN = 4

    def __init__(self, model: "Model", cache, states):
        self.cache_ref = weakref.ref(cache) if cache is not None else None
        self.model_ref = weakref.ref(model)
        order = model.spec.run_order
        sigs, rows = [], []
        self._held = []     # weak references to the layers' own tensors: one that is gone means the table is stale
        for i in range(len(order)):
            ok, scalars, tensors, view = self._entry(model, cache, i)
            planes = sum(1 for t in ((view.k, view.v) if view is not None else ()) if t is not None)
            self._held += [weakref.ref(t) for t in tensors[:len(tensors) - planes]]
            if states is not None and states.tensor(i) is not None:
                ok = False      # state of its own: one tensor per entry that is not on the layer
            sig = (type(model.layers[order[i].layer]), tuple(scalars), tuple((t.shape, t.stride(), t.dtype) for t in tensors),
                   view.group if view is not None else None, view.writes if view is not None else None)
            sigs.append(sig if ok else None)
            rows.append([t.data_ptr() for t in tensors])
        self.run_end: dict[int, int] = {}
        self.table: dict[int, np.ndarray] = {}     # start of a run -> int64 [entries of the run, slots]
        self.plans: dict[tuple, object] = {}       # (start of a run, the recorded calls) -> their list: steps of one shape repeat
        a = 0
        while a < len(order):
            b = a
            while sigs[a] is not None and b + 1 < len(order) and sigs[b + 1] == sigs[a]:
                b += 1
            if b - a + 1 >= max(3, self.MIN_RUN):
                self.run_end[a] = b
                self.table[a] = np.ascontiguousarray(np.asarray(rows[a:b + 1], dtype=np.int64))
            a = b + 1

    def alive(self) -> bool:
        """Whether every tensor whose address the tables hold still exists. (A part binds its tensors once; one
        that replaces a tensor later frees the old one, and the tables are then built anew.)"""
        return all(r() is not None for r in self._held)

    @staticmethod
    def _entry(model, cache, i):
        """(every part launches only, constants, tensors in slot order: the layer's own, then its cache planes,
        the entry's view of the cache)."""
        entry = model.spec.run_order[i]
        tensors, scalars = [], []
        ok = walk_part(model.layers[entry.layer], tensors, scalars, set())
        owner = i if entry.cache_of is None else entry.cache_of
        view = cache.layer_cache(owner, writes=entry.cache_of is None) if cache is not None else None
        tensors += [t for t in ((view.k, view.v) if view is not None else ()) if t is not None]
        return ok, scalars, tensors, view

    def spans(self, i: int, start: int):
        """(address, bytes) per slot of entry i of the run that starts at `start`, looked up afresh; None if
        the layer's tensors are no longer where the table says (then nothing is repeated)."""
        model, cache = self.model_ref(), self.cache_ref() if self.cache_ref is not None else None
        row = self.table[start][i - start]
        _, _, tensors, _ = self._entry(model, cache, i)
        if len(tensors) != len(row) or any(t.data_ptr() != int(p) for t, p in zip(tensors, row)):
            return None
        return [(t.data_ptr(), _extent_bytes(t)) for t in tensors]
