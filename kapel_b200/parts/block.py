"""How a layer's parts are arranged.

"sandwich" (Gemma 2; crates/kapel-models/src/model.rs:1401-1460):
    h = pre_mixer(x); a = mixer(h); x += post_mixer(a); h = pre_ffn(x); m = ffn(h); x += post_ffn(m)
"prenorm": the same without the post norms.

The residual x is float32 and is updated in place. Each sum is one kernel together with the
norm before it and the norm after it, when those are RMS norms.
"""
from __future__ import annotations

from .base import Part
from .norm import add_branch
from .registry import build_part


class SandwichBlock(Part):
    norm_roles = ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")

    @classmethod
    def expected_tensors(cls, spec):
        from .registry import part_class

        out = {}
        out.update(part_class("mixer", spec.mixer.kind).expected_tensors(spec.mixer))
        out.update(part_class("feed_forward", spec.ffn.kind).expected_tensors(spec.ffn))
        for role in cls.norm_roles:
            n = spec.norms[role]
            out.update(part_class("norm", n.kind).expected_tensors(n))
        return out

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        missing = [r for r in self.norm_roles if r not in spec.norms]
        if missing:
            raise ValueError(f"{spec.kind} block: norms {missing} are missing")
        self.mixer = build_part("mixer", spec.mixer, ctx)
        self.ffn = build_part("feed_forward", spec.ffn, ctx)
        self.norms = {r: build_part("norm", spec.norms[r], ctx) for r in self.norm_roles}

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer, self.ffn, *self.norms.values()))

    def cache_needs(self):
        """What this layer keeps between steps: its mixer's pages and state."""
        return self.mixer.cache_needs()

    def first_norm(self):
        """The norm this block applies to the residual first; the block before it may apply it on
        the way and hand the result in as `h`."""
        return self.norms["pre_mixer"]

    def load(self, tensors):
        self.mixer.load(tensors)
        self.ffn.load(tensors)
        for n in self.norms.values():
            n.load(tensors)

    def forward(self, x, h, batch, cache, next_norm):
        if h is None:
            h = self.norms["pre_mixer"].forward(x)
        a = self.mixer.forward(h, batch, cache)
        h = add_branch(self.ctx, x, a, self.norms.get("post_mixer"), self.norms["pre_ffn"])
        m = self.ffn.forward(h)
        h_next = add_branch(self.ctx, x, m, self.norms.get("post_ffn"), next_norm)
        return x, h_next


class PreNormBlock(SandwichBlock):
    norm_roles = ("pre_mixer", "pre_ffn")
