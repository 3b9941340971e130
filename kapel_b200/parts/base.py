"""The interfaces of parts, and what a part is given when it is built and when it runs.

Every part class has:

    expected_tensors(spec) -> {tensor name: shape}      (a static method; no device needed)
    __init__(spec, ctx)                                 (ctx: BuildContext)
    load(tensors)                                       (tensors: a mapping name -> device tensor; it
                                                         may read a tensor only when asked, and may
                                                         offer `copy_into(name, dest)`, `shape(name)`
                                                         and `dtype(name)` as `weights.WeightSource`
                                                         does; `stack_rows` and `matrix_named` below
                                                         use those where they exist)

and, by category:

    norm          forward(x, out_dtype=None) -> y       x float32 or activation dtype, [rows, width]
                  fuse_key() -> a (weight, eps, offset) triple if the fused kernel may apply it, else None
    position      apply(q_and_k ...) is not called by the engine: a mixer owns its position
                  encoding and asks it for what it needs; kind "rope" gives `tables(batch)`.
    mixer         cache_needs() -> CacheNeeds
                  forward(h, batch, cache) -> [rows, hidden] in the activation dtype (or a
                      kernels.SplitSum of that shape, which the block's residual sum adds up)
                      h: [rows, hidden]; batch: engine.batch.StepBatch; cache: LayerCache
    feed_forward  forward(h) -> [rows, hidden] (a tensor or a kernels.SplitSum)
    every part    graph_safe: bool (see `Part`)
    block         forward(x, h, batch, cache, next_norm) -> (x, h_next)
                      x: the float32 residual [rows, hidden] (updated in place);
                      h: this block's first norm already applied to x, or None;
                      next_norm: the norm that the next consumer applies to x first, or None;
                      h_next: next_norm(x) if the block computed it on the way, else None.
                  cache_needs() -> CacheNeeds: what the layer keeps between steps (its mixer's)
                  first_norm() -> the norm the block applies to x first, or None: the block
                      before it may apply it on the way (`next_norm` above)
    embedding     forward(ids) -> float32 [rows, hidden]
    head          forward(x_rows) -> float32 logits [n, vocab]

No part knows which model it is in: sizes and constants come from its spec, tensors by the
names its spec gives.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch


@dataclass
class BuildContext:
    """`dtype` is the activation dtype of the path: bfloat16 (serving) or float32 (everything
    in true 32-bit). `page_size` is the cache's."""

    dtype: torch.dtype
    device: torch.device
    page_size: int = 16
    # weights already prepared for the products, by tensor name: a table that two parts read (a
    # tied embedding and head) is on the device once
    prepared: Dict[str, torch.Tensor] = field(default_factory=dict)

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


class LayerCache:
    """What one layer run sees of the cache: the tables of the layer whose cache it uses, and
    whether it may write them (`owns` is False for a layer that reads another layer's cache)."""

    def __init__(self, manager, cache_layer: int, owns: bool):
        self.manager = manager
        self.layer = cache_layer
        self.owns = owns

    @property
    def group(self) -> int:
        return self.manager.group_of_layer[self.layer]

    def tables(self):
        return self.manager.tables(self.layer)

    def state(self):
        return self.manager.states[self.layer]


class Part:
    # True when `forward` only enqueues kernels whose arguments are device tensors of the batch:
    # such a part can be recorded into a CUDA graph. A part that reads the plan on the host (a
    # loop over requests, say) leaves it False, and the engine then runs every step eagerly. A
    # recorded step may hold rows that belong to no token (padding up to the recording's size):
    # their cache line is -1, and a part must write nothing that lasts for them.
    graph_safe = False

    @staticmethod
    def expected_tensors(spec) -> Dict[str, tuple]:
        return {}

    def __init__(self, spec, ctx: BuildContext):
        self.spec = spec
        self.ctx = ctx

    def load(self, tensors) -> None:
        pass


def matrix_for(ctx: BuildContext, t: torch.Tensor) -> torch.Tensor:
    """A weight as the products take it: kept as stored (bfloat16, or float32 if the file has
    it in 32-bit); widened to float32 on the 32-bit path."""
    if t.device != ctx.device:
        t = t.to(ctx.device)
    if ctx.is_f32 and t.dtype != torch.float32:
        return t.to(torch.float32)
    return t.contiguous()


def matrix_named(ctx: BuildContext, tensors, name: str) -> torch.Tensor:
    """`matrix_for` of the tensor `name`, made once a model: parts that read the same name share it."""
    if name not in ctx.prepared:
        ctx.prepared[name] = matrix_for(ctx, tensors[name])
    return ctx.prepared[name]


def stack_rows(ctx: BuildContext, tensors, names, what: str = "weights") -> torch.Tensor:
    """The matrices `names` (each [rows_i, width]) one below the other in one device tensor, as the
    products take it. Where `tensors` can copy a tensor into a destination (`copy_into`), each
    goes from where it lies (a file's mapping) straight into its rows of the one allocation, so
    the device never holds the parts beside the whole."""
    if hasattr(tensors, "copy_into") and hasattr(tensors, "shape") and hasattr(tensors, "dtype"):
        shapes = [tuple(tensors.shape(n)) for n in names]
        dtypes = {tensors.dtype(n) for n in names}
        parts = None
    else:
        parts = [tensors[n] for n in names]
        shapes = [tuple(p.shape) for p in parts]
        dtypes = {p.dtype for p in parts}
    if len(dtypes) != 1:
        raise ValueError(f"{what}: {', '.join(names)} differ in dtype and cannot be stacked")
    if any(len(s) != 2 or s[1] != shapes[0][1] for s in shapes):
        raise ValueError(f"{what}: {', '.join(names)} have shapes {shapes} and cannot be stacked")
    kept = dtypes.pop()
    dtype = torch.float32 if (ctx.is_f32 and kept.is_floating_point) else kept
    stacked = torch.empty((sum(s[0] for s in shapes), shapes[0][1]), dtype=dtype, device=ctx.device)
    at = 0
    for i, (name, shape) in enumerate(zip(names, shapes)):
        dest = stacked[at : at + shape[0]]
        if parts is None:
            tensors.copy_into(name, dest)
        else:
            dest.copy_(parts[i])
            parts[i] = None
        at += shape[0]
    return stacked


def require_product_widths(ctx: BuildContext, what: str, **widths) -> None:
    """Refuses, when a part is built, inner widths that the bfloat16 products cannot take (their
    rows are read 16 bytes at a time: a multiple of 8 elements), naming the configuration's key.
    The 32-bit path takes any width."""
    if ctx.is_f32:
        return
    bad = {k: v for k, v in widths.items() if v % 8}
    if bad:
        listed = ", ".join(f"{k} = {v}" for k, v in bad.items())
        raise ValueError(f"{what}: {listed} must be a multiple of 8 for the bfloat16 kernels (the float32 path takes any width)")


def linear(ctx: BuildContext, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           softcap: Optional[float] = None, keep_split: bool = False):
    """x . w^T through the library's kernels. A weight kept in 32-bit on the bfloat16 path is
    multiplied in true 32-bit: the input is widened first and the result narrowed after. With
    `keep_split` the result may be a `kernels.SplitSum` (partial sums of a product split over K)
    for a consumer that adds them up itself: `add_branch`, `kernels.glu`, `kernels.rope_append`."""
    from .. import kernels as K

    out_dtype = out_dtype or ctx.dtype
    if w.dtype == torch.float32 and x.dtype != torch.float32:
        x = K.cast(x, torch.float32)
    elif w.dtype == torch.bfloat16 and x.dtype != torch.bfloat16:
        x = K.cast(x, torch.bfloat16)
    return K.gemm(x, w, out_dtype=out_dtype, softcap=softcap, keep_split=keep_split)
