"""Reading and writing safetensors files: 8-byte little-endian header length, a JSON header, raw bytes.

Checks follow the reference's reader (src/model/safetensors.cpp:13-85): supported dtypes,
shapes that do not overflow, `data_offsets` inside the file and equal in size to
shape x dtype; `__metadata__` is skipped. Tensors are views of a memory map; nothing is
copied until a tensor is moved to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

from ..errors import LoadError

# name -> (bytes per element, numpy dtype to view the bytes, torch dtype of the result)
_DTYPES = {
    "F32": (4, np.dtype("<f4"), torch.float32),
    "BF16": (2, np.dtype("<i2"), torch.bfloat16),
    "F16": (2, np.dtype("<f2"), torch.float16),
    "I32": (4, np.dtype("<i4"), torch.int32),
}
_TORCH_TO_NAME = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int32: "I32"}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int   # byte offsets inside the file
    end: int


class SafetensorsFile:
    """One file, memory-mapped read-only. `entries` maps name -> TensorEntry."""

    def __init__(self, path):
        self.path = Path(path)
        try:
            size = self.path.stat().st_size
            f = open(self.path, "rb")
        except OSError as e:
            raise LoadError(f"{self.path}: cannot open ({e.strerror})") from None
        with f:
            if size == 0:
                raise LoadError(f"{self.path}: file is empty")
            if size < 8:
                raise LoadError(f"{self.path}: truncated header length")
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > size - 8:
            raise LoadError(f"{self.path}: header of {hlen} bytes runs past the end of the file")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise LoadError(f"{self.path}: invalid JSON header: {e}") from None
        if not isinstance(header, dict):
            raise LoadError(f"{self.path}: header is not a JSON object")
        data_start, data_size = 8 + hlen, size - 8 - hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype, shape, (b, e) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise LoadError(f"{self.path}: tensor '{name}' has a malformed header entry") from None
            if dtype not in _DTYPES:
                raise LoadError(f"{self.path}: tensor '{name}' has unsupported dtype {dtype} (supported: "
                                f"{', '.join(_DTYPES)})")
            if any((not isinstance(d, int)) or d < 0 for d in shape):
                raise LoadError(f"{self.path}: tensor '{name}' has a bad shape {list(shape)}")
            numel = 1
            for d in shape:
                numel *= d
                if numel > 2 ** 62:
                    raise LoadError(f"{self.path}: tensor '{name}' has an overflowing shape {list(shape)}")
            if not (isinstance(b, int) and isinstance(e, int) and 0 <= b <= e <= data_size):
                raise LoadError(f"{self.path}: tensor '{name}' has data_offsets [{b}, {e}] outside the {data_size} data bytes")
            if e - b != numel * _DTYPES[dtype][0]:
                raise LoadError(f"{self.path}: tensor '{name}' holds {e - b} bytes but shape {list(shape)} of {dtype} "
                                f"needs {numel * _DTYPES[dtype][0]}")
            self.entries[name] = TensorEntry(name, dtype, shape, data_start + b, data_start + e)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (bfloat16 stays bfloat16, 32-bit stays 32-bit)."""
        e = self.entries[name]
        _, np_dtype, torch_dtype = _DTYPES[e.dtype]
        arr = np.frombuffer(self._map, dtype=np_dtype, count=(e.end - e.begin) // np_dtype.itemsize, offset=e.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the tensor is only ever copied from
            t = torch.from_numpy(arr)
        if torch_dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(e.shape)


def write_safetensors(path, tensors: dict[str, torch.Tensor]) -> None:
    header, offset = {}, 0
    for name, t in tensors.items():
        if t.dtype not in _TORCH_TO_NAME:
            raise LoadError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for t in tensors.values():
            c = t.detach().cpu().contiguous()
            if c.dtype == torch.bfloat16:
                c = c.view(torch.int16)
            f.write(c.numpy().tobytes())
