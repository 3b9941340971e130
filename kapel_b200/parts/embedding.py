"""The two ends of the model: token rows times a scale in, soft-capped logits out.

x = table[ids] * scale, the scale rounded to the activation dtype as Kapel rounds it
(crates/kapel-models/src/model.rs:633,653-656,2079-2083). logits = cap * tanh((h . table^T) / cap)
on the rows asked for (model.rs:1355-1381); here the product, the cap and the widening to
float32 are one kernel, so the logits are not rounded to the activation dtype on the way.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, linear, matrix_named


class Embedding(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        return {}          # the table's shape is the model's [vocab, hidden]; ModelParts adds it

    def load(self, tensors):
        self.table = matrix_named(self.ctx, tensors, self.spec.weight)
        scale = float(self.spec.scale)
        if self.spec.round_scale and self.ctx.dtype == torch.bfloat16:
            scale = float(torch.tensor(scale, dtype=torch.float32).to(torch.bfloat16).float())
        elif self.spec.round_scale:
            scale = float(torch.tensor(scale, dtype=torch.float32))
        self.scale = scale

    def forward(self, ids):
        return K.embed(self.table, ids, self.scale)


class VocabHead(Part):
    graph_safe = True

    def load(self, tensors):
        self.table = matrix_named(self.ctx, tensors, self.spec.weight)

    def forward(self, h):
        return linear(self.ctx, h, self.table, out_dtype=torch.float32, softcap=self.spec.softcap)
