"""Weights by tensor name, checked against what the model's parts expect, all at once.

Kapel reads every tensor of the checkpoint into a map by name and reports a missing weight at
first use (crates/kapel-models/src/model.rs:294-311,581-585). Here the parts say up front which
names and shapes they read (`parts.expected_tensors`), and one error lists everything that is
missing or of the wrong shape, and the tensors of the file that the model does not name. As in
Kapel, only the names the model reads are required: a file may hold more (another head, a
vision tower), and such tensors alone are no error unless the caller asks for `strict`; they
are listed in the error when there is one, and kept in `WeightSource.unexpected`.

A folder is opened as a `WeightSource`: a mapping from name to tensor that reads nothing until
it is asked. `source[name]` puts one tensor on the device; `source.copy_into(name, dest)` copies
it from the file's mapping straight into `dest`, a part of a larger device tensor, which is how
the stacked q|k|v and gate|up weights are made without ever holding their parts on the device
(Kapel drops the parts as it stacks them, model.rs:415-480).

Float tensors stay as the file has them when that is bfloat16 or float32 (float16 and float64
become bfloat16 and float32); integer tables become int32. The 32-bit path widens on the
device, in the parts.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Iterator, List, Mapping, Tuple

import torch

from .safetensors import SafetensorsError, SafetensorsFile


class WeightsError(ValueError):
    """The file's tensors are not the model's; `.missing`, `.unexpected`, `.wrong_shape` say how."""

    def __init__(self, missing, unexpected, wrong_shape, source=""):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights of {source} do not fit the model:" if source else "weights do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(
                f"  wrong shape ({len(self.wrong_shape)}): "
                + ", ".join(f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape)
            )
        super().__init__("\n".join(lines))


def _canonical(name: str) -> str:
    """`model.language_model.X` is `model.X` (crates/kapel-models/src/model.rs:2019-2035)."""
    if name.startswith("model.language_model."):
        return "model." + name[len("model.language_model."):]
    return name


def check_names(expected: Mapping[str, tuple], found: Mapping[str, tuple], source: str = "", strict: bool = True) -> List[str]:
    """Raises one `WeightsError` if a name is missing or a shape is wrong (and, with `strict`, if
    the file holds a tensor the model does not name); returns the unexpected names otherwise."""
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted((n, tuple(found[n]), tuple(expected[n])) for n in expected if n in found and tuple(found[n]) != tuple(expected[n]))
    if missing or wrong or (strict and unexpected):
        raise WeightsError(missing, unexpected, wrong, source)
    return unexpected


def _kept_dtype(dtype: torch.dtype) -> torch.dtype:
    if dtype in (torch.bfloat16, torch.float32):
        return dtype
    if dtype == torch.float16:
        return torch.bfloat16
    if dtype == torch.float64:
        return torch.float32
    if dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return torch.int32
    raise WeightsError([], [], [], f"a tensor of dtype {dtype}")


def open_files(folder):
    """The safetensors files of a model folder: `model.safetensors`, or the shards its index names
    (crates/kapel-hub/src/checkpoint.rs:47-89)."""
    folder = Path(folder)
    single = folder / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text()).get("weight_map", {})
        names = sorted(set(weight_map.values()))
        for n in names:
            if "/" in n or "\\" in n or n.startswith("."):
                raise SafetensorsError(f"{index}: shard name {n!r} is not a plain file name")
        return [SafetensorsFile(folder / n) for n in names]
    raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


class WeightSource(Mapping):
    """The tensors of a model folder by (canonical) name, read when asked for.

    `shapes()` costs nothing (the files' headers); `source[name]` is that tensor on `device` in
    its kept dtype, a new copy at every call; `copy_into(name, dest)` copies it into `dest` (any
    device, any float dtype) without a device tensor of its own in between. `check(expected)`
    compares the headers with what a model reads and remembers the `unexpected` names.
    """

    def __init__(self, folder, device):
        self.folder = Path(folder)
        self.device = device
        self.files = open_files(folder)
        self._where: Dict[str, Tuple[SafetensorsFile, str]] = {}
        for f in self.files:
            for raw in f.names():
                self._where[_canonical(raw)] = (f, raw)
        self.unexpected: List[str] = []

    # ---- the mapping
    def __iter__(self) -> Iterator[str]:
        return iter(self._where)

    def __len__(self) -> int:
        return len(self._where)

    def __contains__(self, name) -> bool:
        return name in self._where

    def __getitem__(self, name) -> torch.Tensor:
        t = self.host(name)
        return t.to(device=self.device, dtype=_kept_dtype(t.dtype))

    # ---- without reading
    def shape(self, name) -> Tuple[int, ...]:
        f, raw = self._where[name]
        return tuple(f.shape(raw))

    def dtype(self, name) -> torch.dtype:
        f, raw = self._where[name]
        return _kept_dtype(f.dtype(raw))

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {n: tuple(f.shape(raw)) for n, (f, raw) in self._where.items()}

    def check(self, expected: Mapping[str, tuple], strict: bool = False) -> List[str]:
        self.unexpected = check_names(expected, self.shapes(), str(self.folder), strict)
        return self.unexpected

    # ---- reading
    def host(self, name) -> torch.Tensor:
        """The tensor as the file has it: a read-only view of the mapping on the CPU."""
        f, raw = self._where[name]
        return f.tensor(raw)

    def copy_into(self, name, dest: torch.Tensor) -> None:
        """`dest` (of the tensor's shape) receives the tensor, converted to dest's dtype."""
        t = self.host(name)
        if tuple(t.shape) != tuple(dest.shape):
            raise WeightsError([], [], [(name, tuple(t.shape), tuple(dest.shape))], str(self.folder))
        kept = _kept_dtype(t.dtype)
        if t.dtype != kept:
            t = t.to(kept)                  # float16 -> bfloat16 and the like, on the host
        dest.copy_(t)

    def close(self) -> None:
        for f in self.files:
            f.close()


def open_weights(folder, device) -> WeightSource:
    return WeightSource(folder, device)


def load_tensors(folder, expected: Mapping[str, tuple], device, strict: bool = False) -> Dict[str, torch.Tensor]:
    """Every expected tensor of the folder on `device`, all at once; raises `WeightsError` listing
    all faults. (The engine itself loads through a `WeightSource`, tensor by tensor.)"""
    source = WeightSource(folder, device)
    source.check(expected, strict)
    out = {name: source[name] for name in expected}
    source.close()
    return out
