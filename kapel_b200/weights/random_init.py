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
from typing import Dict

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


def random_tensors(config, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    from ..parts import expected_tensors

    spec = config.to_spec()
    return {
        name: random_tensor(name, shape, config.init_std(name, shape), seed, device, dtype)
        for name, shape in expected_tensors(spec).items()
    }


def write_random_model(folder, config, seed: int, dtype=torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config` with weights from `seed`."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config.to_json(), indent=2))
    write_safetensors(folder / "model.safetensors", random_tensors(config, seed, "cpu", dtype),
                      metadata={"format": "pt", "seed": seed})
    return folder
