"""A model as built parts, and its forward pass over one step's rows.

The order of layers is the spec's `schedule`: a list of (layer, whose cache), so a layer may
run twice or read another layer's keys and values. Kapel's forward pass is
crates/kapel-models/src/model.rs:1272-1383: embed, blocks, the rows wanted, final norm, head.
"""
from __future__ import annotations

from typing import Dict, List, Mapping

import torch

from .. import kernels as K
from ..cache import CacheNeeds
from ..parts import BuildContext, LayerCache, build_part, expected_tensors


class ModelParts:
    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx
        for e in spec.schedule:
            if not (0 <= e.layer < len(spec.layers) and 0 <= e.cache_of < len(spec.layers)):
                raise ValueError(f"schedule entry {e} names a layer outside 0..{len(spec.layers) - 1}")
        self.embedding = build_part("embedding", spec.embed, ctx)
        self.blocks = [build_part("block", layer, ctx) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, ctx)
        self.head = build_part("head", spec.head, ctx)

    def expected_tensors(self) -> Dict[str, tuple]:
        return expected_tensors(self.spec)

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.embedding.load(tensors)
        for b in self.blocks:
            b.load(tensors)
        self.final_norm.load(tensors)
        self.head.load(tensors)

    def graph_safe(self) -> bool:
        """Whether every part only enqueues kernels, so that a decode step can be recorded."""
        return all(p.graph_safe for p in (self.embedding, self.final_norm, self.head, *self.blocks))

    def cache_needs(self) -> Dict[int, CacheNeeds]:
        """What each cache-owning layer keeps: layers named as `cache_of` in the schedule."""
        owners = sorted({e.cache_of for e in self.spec.schedule})
        return {l: self.blocks[l].cache_needs() for l in owners}

    def forward(self, batch, cache_manager) -> torch.Tensor:
        """float32 logits [wanted rows, vocab] of a step."""
        x = self.embedding.forward(batch.ids)
        schedule = self.spec.schedule
        h = None
        for i, e in enumerate(schedule):
            block = self.blocks[e.layer]
            nxt = self.blocks[schedule[i + 1].layer].first_norm() if i + 1 < len(schedule) else None
            cache = LayerCache(cache_manager, e.cache_of, owns=(e.cache_of == e.layer))
            x, h = block.forward(x, h, batch, cache, nxt)
        rows = K.gather_rows(x, batch.want_rows)
        return self.head.forward(self.final_norm.forward(rows))
