"""Position encodings. A mixer owns one and asks it for what its kernels take.

kind "rope": theta^(-2j/r) frequencies, pairing (j, j + r/2), all in one table of (cos, sin)
per row made once a step with angles in 64-bit (crates/kapel-ops/src/rope.rs:63-101;
kernels/src/lib.rs rope_table :1092). kind "none": no rotation.
"""
from __future__ import annotations

from .. import kernels as K
from .base import Part


class Rope(Part):
    graph_safe = True

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.pairing != "half":
            raise ValueError(f"rope pairing {spec.pairing!r} is not built (only \"half\")")
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rope rotary_dim {spec.rotary_dim} must be positive and even")

    @property
    def rotary_dim(self) -> int:
        return self.spec.rotary_dim

    def tables(self, batch):
        """(cos, sin) [rows, rotary/2, 2] for this step's positions; shared by every layer with
        the same theta and rotary width."""
        key = ("rope", float(self.spec.theta), int(self.spec.rotary_dim))
        if key not in batch.memo:
            batch.memo[key] = K.rope_table(batch.positions, self.spec.rotary_dim, self.spec.theta)
        return batch.memo[key]


class NoPosition(Part):
    graph_safe = True

    rotary_dim = 0

    def tables(self, batch):
        return None
