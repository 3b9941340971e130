"""RMS norm with an offset on its weight: y = x / sqrt(mean(x^2) + eps) * (offset + w)
(crates/kapel-ops/src/norm.rs:123-135; Gemma 2's offset is 1, crates/kapel-models/src/config.rs:284)."""
from __future__ import annotations

from .. import kernels as K
from .base import Part


class RMSNorm(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        return {spec.weight: (spec.width,)}

    def load(self, tensors):
        w = tensors[self.spec.weight]
        if w.device != self.ctx.device:
            w = w.to(self.ctx.device)
        self.weight = w.float() if self.ctx.is_f32 else w.contiguous()

    def forward(self, x, out_dtype=None):
        return K.rmsnorm(x, self.weight, self.spec.eps, self.spec.offset, out_dtype or self.ctx.dtype)

    def fuse_key(self):
        """(weight, eps, offset): what the fused add-and-norm kernel needs to apply this norm."""
        return (self.weight, self.spec.eps, self.spec.offset)


def add_branch(ctx, residual, branch, post_norm, next_norm):
    """residual += post_norm(branch) (post_norm None: plain sum); returns next_norm(residual),
    or None without a next norm. One kernel when the norms are RMS norms with weights of one
    dtype; a norm of another kind runs through its own `forward` around the fused sum."""
    post_key = post_norm.fuse_key() if hasattr(post_norm, "fuse_key") else None
    next_key = next_norm.fuse_key() if hasattr(next_norm, "fuse_key") else None
    if post_norm is not None and post_key is None:
        branch = post_norm.forward(K.finish(branch, ctx.dtype))
    if next_key is not None and (post_key is None or post_key[0].dtype == next_key[0].dtype):
        return K.add_rmsnorm(residual, branch, post_key, next_key, ctx.dtype)
    K.add_rmsnorm(residual, branch, post_key, None, ctx.dtype)
    return next_norm.forward(residual) if next_norm is not None else None
