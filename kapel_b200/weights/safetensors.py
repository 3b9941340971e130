"""Reading and writing safetensors files, by tensor name.

The format, as Kapel checks it (crates/kapel-hub/src/safetensors.rs:110-204): eight bytes of
little-endian header length (at most 100 MB), a JSON object name -> {dtype, shape,
data_offsets}, then the bytes; offsets must lie inside the file, agree with shape and dtype,
and not overlap the header. A file is mapped, not read: a tensor is a view of the mapping
until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_MAX_HEADER = 100 * 1024 * 1024

_DTYPES = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors file; the message says where."""


class SafetensorsFile:
    """One mapped file: `names()`, `shape(name)`, `dtype(name)`, `tensor(name)`."""

    def __init__(self, path):
        self.path = Path(path)
        if not self.path.is_file():
            raise SafetensorsError(f"{self.path}: no such file")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: {size} bytes is too short for a header length")
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{self.path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._map[8 : 8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", None)
        self._base = 8 + n
        data_size = size - self._base
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            try:
                kind, shape, (a, b) = meta["dtype"], tuple(meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: entry {name!r} lacks dtype, shape or data_offsets") from None
            if kind not in _DTYPES:
                raise SafetensorsError(f"{self.path}: {name!r} has dtype {kind!r}, which this reader does not take")
            if any((not isinstance(s, int)) or s < 0 for s in shape):
                raise SafetensorsError(f"{self.path}: {name!r} has shape {list(shape)}")
            count = 1
            for s in shape:
                count *= s
            want = count * _DTYPES[kind][1]
            if not (isinstance(a, int) and isinstance(b, int)) or a < 0 or b < a or b > data_size:
                raise SafetensorsError(f"{self.path}: {name!r} offsets [{a}, {b}) lie outside the data ({data_size} bytes)")
            if b - a != want:
                raise SafetensorsError(
                    f"{self.path}: {name!r} holds {b - a} bytes, but {kind}{list(shape)} needs {want}"
                )
            self._entries[name] = (kind, shape, a, b)

    def names(self) -> Iterable[str]:
        return self._entries.keys()

    def __contains__(self, name) -> bool:
        return name in self._entries

    def shape(self, name) -> Tuple[int, ...]:
        return self._entries[name][1]

    def dtype(self, name) -> torch.dtype:
        return _DTYPES[self._entries[name][0]][0]

    def tensor(self, name) -> torch.Tensor:
        """A read-only view of the mapping as a CPU tensor (copy it before writing)."""
        kind, shape, a, b = self._entries[name]
        dt = _DTYPES[kind][0]
        if b == a:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._map)[self._base + a : self._base + b]
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")       # torch warns that the buffer is read-only
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(shape)

    def close(self):
        # Tensors handed out keep the mapping alive through their buffers; closing the file
        # handle is all that is needed.
        try:
            self._file.close()
        except Exception:
            pass


def write_safetensors(path, tensors: Dict[str, torch.Tensor], metadata=None) -> None:
    """Writes `tensors` (CPU, any of the dtypes above) under their names, sorted by name."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name!r}: dtype {t.dtype} cannot be written")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel() == 0:
                continue
            raw = t.view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
            f.write(memoryview(raw.reshape(-1).numpy()))
