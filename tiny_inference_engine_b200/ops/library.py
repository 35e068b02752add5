"""Loads the engine's CUDA library (compiling it at first use) and declares its entry points.

There is no CPU fallback and no library attention or model code behind these functions: if the
library cannot be built or loaded, or the GPU is not the one it was compiled for, the engine
stops with an error that says so.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

_LOCK = threading.Lock()
_LIB = None

P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES = {
    "tie_embed": [I, P, P, P, I, I, I, I, P],
    "tie_scatter_ids": [P, P, P, P, I, P],
    "tie_add_rmsnorm": [I, P, P, P, L, I, P, P, F, P, I, I, P],
    "tie_rmsnorm_rows": [I, P, L, P, F, P, L, I, L, P],
    "tie_silu_mul": [I, P, P, I, I, P],
    "tie_rope": [I, P, L, P, P, I, I, I, I, P],
    "tie_kv_append": [I, P, P, L, L, P, P, P, I, I, I, I, P],
    "tie_qk_norm_rope_append": [I, P, L, P, L, I, L, P, P, F, F, P, I, P, P, P, P, I, I, I, I, I, I, P],
    "tie_gemm_simt": [I, I, P, P, P, I, I, I, L, L, L, P],
    "tie_attention_rows": [I, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "tie_attention_split": [I, P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, I, I, I, P, P],
    "tie_sample": [P, L, I, I, P, P, P, P, P],
    "tie_sample_filtered": [P, L, I, I, P, P, P, P, P, P, I, P],
    "tie_gemm_tc": [I, P, P, P, I, I, I, L, L, L, I, I, I, P, I, I, I, I, I, P],
    "tie_gemm_tc2": [I, P, P, P, I, I, I, L, L, L, I, I, I, I, P],
    "tie_attention_prompt_tc": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P],
    "tie_attention_decode_tc": [P, L, P, P, P, P, P, I, I, I, I, I, I, F, P, I, I, I, P, P],
    "tie_attention_decode_tma": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, I, I, I, I, P, P, I, P],
    "tie_attention_decode_prep": [P, L, P, L, I, L, P, P, F, F, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, I, I, I, I, P, P, I, P],
    "tie_attention_prompt_tma": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
    "tie_attention_prompt_umma": [P, L, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
    "tie_attention_merge": [I, P, P, P, I, I, I, P, I, I, I, P, P],
}


class KernelLibraryError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The loaded library; built on first call."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        from ..csrc.build import build
        try:
            path = build()
        except Exception as e:  # no nvcc, compile error: never continue without the kernels
            raise KernelLibraryError(f"the engine's CUDA kernels could not be built: {e}") from e
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelLibraryError(f"the engine's CUDA library {path} could not be loaded: {e}") from e
        lib.tie_last_error.restype = ctypes.c_char_p
        lib.tie_last_error.argtypes = []
        lib.tie_compiled_arch.restype = c_int
        lib.tie_kernel_status.restype = c_int
        lib.tie_kernel_status.argtypes = []
        lib.tie_gemm_tc_real_splits.restype = c_int
        lib.tie_gemm_tc_real_splits.argtypes = [c_int, c_int]
        lib.tie_attention_decode_limit.restype = c_int
        lib.tie_attention_decode_limit.argtypes = [c_int]
        lib.tie_gemm_tc2_pairs.restype = c_int
        lib.tie_gemm_tc2_pairs.argtypes = []
        lib.tie_replay_launcher_id.restype = c_int
        lib.tie_replay_launcher_id.argtypes = [ctypes.c_char_p]
        lib.tie_replay_launcher_args.restype = c_int
        lib.tie_replay_launcher_args.argtypes = [c_int]
        lib.tie_replay_layers.restype = c_int
        lib.tie_replay_layers.argtypes = [P, P, P, P, P, I, P, I, I, P]
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = c_int
        _LIB = lib
        return lib


def register_signature(name: str, argtypes: list) -> None:
    """Declares an entry point added by another source file of the library."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def check_device() -> None:
    """The kernels are sm_100a code: refuse any other GPU, and a machine without one, loudly."""
    import torch
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: this engine runs on a B200 only and has no CPU path")
    major, minor = torch.cuda.get_device_capability()
    if major * 10 + minor != library().tie_compiled_arch():
        raise KernelLibraryError(f"the kernels are compiled for sm_100a, this GPU is sm_{major}{minor}")


_LAUNCHES = 0


def launch_count() -> int:
    """How many launcher calls this process has made (each launches one to three kernels of this library)."""
    return _LAUNCHES


_ENTRY: dict = {}     # name -> bound entry point (looked up once: eager steps make hundreds of calls)
_RECORDING = None     # a list while ops/replay.py records the calls of one layer


def call(name: str, *args) -> None:
    global _LAUNCHES
    fn = _ENTRY.get(name)
    if fn is None:
        fn = _ENTRY[name] = getattr(library(), name)
    _LAUNCHES += 1
    status = fn(*args)
    if status != 0:
        from ..errors import InvalidArgument, TieError
        msg = library().tie_last_error().decode()
        raise (InvalidArgument if status == 1 else TieError)(msg)
    if _RECORDING is not None:
        _RECORDING.append((name, args))
