"""Random weights from a configuration and a seed, and a model folder made of them.

Kapel's inference side has no such mode; its training `init` seeds each tensor by
FNV-1a(name) xor seed (crates/kapel-train/src/model.rs:932-961). The same idea here: every tensor
has a generator of its own, keyed by its name, so the values do not depend on the order in
which tensors are made or on which of them are made. Standard deviations come from the
configuration class (`init_std(name, shape)`).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from .safetensors import write_safetensors


def _fnv1a(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def tensor_seed(name: str, seed: int) -> int:
    return (_fnv1a(name) ^ (seed & 0xFFFFFFFFFFFFFFFF)) & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, shape, std: float, seed: int, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    """N(0, std) values for tensor `name`, rounded to `dtype`. The CPU and the CUDA generators
    differ, so a folder written on the CPU is what both a test's plain implementation and the
    engine read; on a CUDA device this is for timing runs, where only the shapes matter."""
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(name, seed))
    t = torch.empty(tuple(shape), dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype)


class RandomSource(Mapping):
    """The random tensors of a configuration by name, each made when it is asked for (on `device`),
    so that a model of any size can be built without its parts lying about twice. The interface is
    `weights.WeightSource`'s."""

    def __init__(self, config, seed: int, device="cpu", dtype=torch.bfloat16):
        from ..parts import expected_tensors

        self.config, self.seed, self.device, self._dtype = config, seed, device, dtype
        self._shapes = {n: tuple(s) for n, s in expected_tensors(config.to_spec()).items()}
        self.unexpected = []

    def __iter__(self):
        return iter(self._shapes)

    def __len__(self):
        return len(self._shapes)

    def __contains__(self, name):
        return name in self._shapes

    def __getitem__(self, name):
        shape = self._shapes[name]
        return random_tensor(name, shape, self.config.init_std(name, shape), self.seed, self.device, self._dtype)

    def shape(self, name):
        return self._shapes[name]

    def dtype(self, name):
        return self._dtype

    def shapes(self):
        return dict(self._shapes)

    def check(self, expected, strict: bool = False):
        from .loader import check_names

        return check_names(expected, self._shapes, "random weights", strict)

    def copy_into(self, name, dest) -> None:
        dest.copy_(self[name])

    def close(self) -> None:
        pass


def random_tensors(config, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    from ..parts import expected_tensors

    spec = config.to_spec()
    return {
        name: random_tensor(name, shape, config.init_std(name, shape), seed, device, dtype)
        for name, shape in expected_tensors(spec).items()
    }


def write_random_model(folder, config, seed: int, dtype=torch.bfloat16, device="cpu") -> Path:
    """Writes config.json and model.safetensors for `config` with weights from `seed`. `device` is
    where the values are drawn before they are written: a CUDA device makes a folder of several GB
    in seconds (its generator gives other values than the CPU's for the same seed; the folder, not
    the seed, is then what its readers share)."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=2))
    write_safetensors(folder / "model.safetensors", random_tensors(config, seed, device, dtype),
                      metadata={"format": "pt", "seed": seed})
    return folder
