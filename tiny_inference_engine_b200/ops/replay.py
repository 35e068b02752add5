"""Records the launcher calls of one layer and repeats them for the layers after it that are built alike.

A step that is not a captured graph makes about eight launcher calls per layer from Python; for a
few hundred tokens the GPU is done with a layer before the host has issued the next one. Layers
that are built alike make the same calls with the same arguments except for the addresses of
their own tensors. `record()` collects the calls of one layer; `plan()` marks every pointer argument (known
from the launcher's declared signature) that points into one of that layer's tensors as (slot, offset within it); `run()` hands the list and a
table of the following layers' addresses to `tie_replay_layers` (csrc/layer_replay.cu), which
issues the same launchers with the same arguments: one call from Python for all of them.
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager
from dataclasses import dataclass

import numpy as np

from . import library



@contextmanager
def record():
    """Collects (name, args) of every launcher call made inside the block."""
    calls: list = []
    previous, library._RECORDING = library._RECORDING, calls
    try:
        yield calls
    finally:
        library._RECORDING = previous


@dataclass
class ReplayPlan:
    fn: np.ndarray          # int32 [calls]: index of the launcher
    arg_begin: np.ndarray   # int32 [calls + 1]
    words: np.ndarray       # int64: every argument, floats as the bits of a double
    slot: np.ndarray        # int32 per argument: -1, or which of the layer's tensors it points into
    offset: np.ndarray      # int64 per argument: bytes from the start of that tensor
    calls: int
    slots_used: tuple       # slots that some argument names


def plan(calls, spans) -> ReplayPlan | None:
    """`calls`: what `record()` collected. `spans`: (address, bytes) of each tensor of the recorded layer, in
    slot order; the first span that contains an address wins, and the same rule holds for every layer, whose
    tensors are laid out alike. None if a call is not one that the library can repeat."""
    lib = library.library()
    fn, begin, words, slot, offset = [], [0], [], [], []
    for name, args in calls:
        fid = lib.tie_replay_launcher_id(name.encode())
        kinds = library._SIGNATURES.get(name)
        if fid < 0 or lib.tie_replay_launcher_args(fid) != len(args) or kinds is None or len(kinds) != len(args):
            return None
        fn.append(fid)
        for a, kind in zip(args, kinds):
            s, off = -1, 0
            if a is None:
                w = 0
            elif isinstance(a, float):
                w = int(np.float64(a).view(np.int64))
            else:
                w = int(a)
                if kind is library.P and w != 0:        # a pointer by the launcher's own signature, not by its size
                    for i, (base, nbytes) in enumerate(spans):
                        if base <= w < base + nbytes:
                            s, off = i, w - base
                            break
            words.append(w)
            slot.append(s)
            offset.append(off)
        begin.append(len(words))
    return ReplayPlan(np.asarray(fn, np.int32), np.asarray(begin, np.int32), np.asarray(words, np.int64),
                      np.asarray(slot, np.int32), np.asarray(offset, np.int64), len(fn),
                      tuple(sorted({s for s in slot if s >= 0})))


_FAILED_AT = ctypes.c_int(0)
layers_repeated = 0     # how many layers this process has issued through `run` (tests and statistics)


def run(p: ReplayPlan, layer_ptrs: np.ndarray) -> None:
    """Repeats the plan once per row of `layer_ptrs` (int64 [layers, slots], contiguous)."""
    global layers_repeated
    layers, slots = layer_ptrs.shape
    if layers == 0 or p.calls == 0:
        return
    lib = library.library()
    _FAILED_AT.value = 0
    status = lib.tie_replay_layers(p.fn.ctypes.data, p.arg_begin.ctypes.data, p.words.ctypes.data, p.slot.ctypes.data,
                                   p.offset.ctypes.data, p.calls, layer_ptrs.ctypes.data, slots, layers,
                                   ctypes.byref(_FAILED_AT))
    if status != 0:
        from ..errors import InvalidArgument, TieError
        msg = lib.tie_last_error().decode()
        done = _FAILED_AT.value
        library._LAUNCHES += done
        raise (InvalidArgument if status == 1 else TieError)(
            f"{msg} (repeating call {done % p.calls} of a recorded layer, {done // p.calls} layers after it)")
    library._LAUNCHES += layers * p.calls
    layers_repeated += layers
