"""The gated feed-forward: down(act(gate(h)) * up(h)), gate and up as one stacked product
(crates/kapel-models/src/model.rs:1429-1456; the gated unit kernels/src/lib.rs glu_any :2489)."""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, linear, matrix_named, require_product_widths, stack_rows


class GatedMLP(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        w = spec.weights
        return {
            w["gate"]: (spec.intermediate, spec.hidden),
            w["up"]: (spec.intermediate, spec.hidden),
            w["down"]: (spec.hidden, spec.intermediate),
        }

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.activation not in K.ACT_CODES:
            raise ValueError(f"gated_mlp: activation {spec.activation!r} is not built")
        require_product_widths(ctx, "gated_mlp", hidden_size=spec.hidden, intermediate_size=spec.intermediate)

    def load(self, tensors):
        w = self.spec.weights
        self.w_gate_up = stack_rows(self.ctx, tensors, [w["gate"], w["up"]], "gated_mlp")
        self.w_down = matrix_named(self.ctx, tensors, w["down"])

    def forward(self, h):
        # many rows of bfloat16: the gated unit is the epilogue of the gate|up product
        inner = K.gemm_glu_fused(h, self.w_gate_up, self.spec.activation) if h.dtype == self.w_gate_up.dtype else None
        if inner is None:
            gu = linear(self.ctx, h, self.w_gate_up, keep_split=True)
            inner = K.glu(gu, self.spec.activation, out_dtype=self.ctx.dtype)
        return linear(self.ctx, inner, self.w_down, keep_split=True)
