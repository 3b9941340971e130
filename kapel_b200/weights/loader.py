"""Weights by tensor name, checked against what the model's parts expect, all at once.

Kapel reads every tensor of the checkpoint into a map by name and reports a missing weight at
first use (crates/kapel-models/src/model.rs:294-311,581-585). Here the parts say up front which
names and shapes they read (`parts.expected_tensors`), and one error lists everything that is
missing, unexpected, or of the wrong shape.

Float tensors stay as the file has them when that is bfloat16 or float32 (float16 and float64
become bfloat16 and float32); integer tables become int32. The 32-bit path widens on the
device, in the parts.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Mapping

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


def check_names(expected: Mapping[str, tuple], found: Mapping[str, tuple], source: str = "") -> None:
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected)
    wrong = sorted((n, tuple(found[n]), tuple(expected[n])) for n in expected if n in found and tuple(found[n]) != tuple(expected[n]))
    if missing or unexpected or wrong:
        raise WeightsError(missing, unexpected, wrong, source)


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


def load_tensors(folder, expected: Mapping[str, tuple], device) -> Dict[str, torch.Tensor]:
    """Every expected tensor of the folder on `device`; raises `WeightsError` listing all faults."""
    files = open_files(folder)
    where = {}
    for f in files:
        for raw in f.names():
            where[_canonical(raw)] = (f, raw)
    check_names(expected, {n: f.shape(raw) for n, (f, raw) in where.items()}, str(folder))
    out = {}
    for name in expected:
        f, raw = where[name]
        t = f.tensor(raw)
        out[name] = t.to(device=device, dtype=_kept_dtype(t.dtype))
    for f in files:
        f.close()
    return out
