"""Grouped-query attention over the paged cache.

q, k, v come from one stacked product (Kapel stacks them at load: crates/kapel-models/src/model.rs:415-480,
1506-1517); one kernel rotates q and k and appends k and v to the cache at the rows' lines
(Kapel: rope_any twice and write_rows_any twice, model.rs:1561-1579); attention reads the pages
through the block table with scale, soft cap and window as arguments (model.rs:1580-1590);
then the output product (model.rs:1633-1637).
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..cache import CacheNeeds, PagedKV
from .base import Part, linear, matrix_named, require_product_widths, stack_rows
from .registry import build_part


class Attention(Part):
    graph_safe = True

    @staticmethod
    def expected_tensors(spec):
        qd, kvd = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        w = spec.weights
        return {w["q"]: (qd, spec.hidden), w["k"]: (kvd, spec.hidden), w["v"]: (kvd, spec.hidden), w["o"]: (spec.hidden, qd)}

    def __init__(self, spec, ctx):
        super().__init__(spec, ctx)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"attention: {spec.num_heads} heads over {spec.num_kv_heads} kv heads")
        if spec.head_dim % 16:
            raise ValueError(f"attention: head_dim {spec.head_dim} must be a multiple of 16 for the kernels")
        require_product_widths(ctx, "attention", hidden_size=spec.hidden,
                               **{"num_attention_heads x head_dim": spec.num_heads * spec.head_dim})
        self.position = build_part("position", spec.position, ctx)

    def load(self, tensors):
        w = self.spec.weights
        self.w_qkv = stack_rows(self.ctx, tensors, [w["q"], w["k"], w["v"]], "attention")
        self.w_o = matrix_named(self.ctx, tensors, w["o"])

    def cache_needs(self) -> CacheNeeds:
        s = self.spec
        return CacheNeeds(paged=PagedKV(s.num_kv_heads, s.head_dim, s.window))

    def forward(self, h, batch, cache):
        s = self.spec
        qkv = linear(self.ctx, h, self.w_qkv, keep_split=True)
        k_table, v_table = cache.tables()
        group = batch.groups[cache.group]
        heads_per_kv = s.num_heads // s.num_kv_heads
        if K.attention_decode_fused_takes(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.position.rotary_dim,
                                          self.ctx.page_size, self.ctx.dtype):
            decode, tiles, split, slots, relative = batch.attention_tiles(
                heads_per_kv, s.num_kv_heads, s.window, s.head_dim,
                K.attention_prompt_kernel(s.num_heads, s.num_kv_heads, s.head_dim, self.ctx.page_size, s.softcap))
            if decode and relative:         # every request brings one token: rotation, the cache's new line and attention in one kernel
                y = K.paged_attention_decode_fused(
                    qkv, self.position.tables(batch), group.lines, k_table, v_table, group.block_table, batch.row_count,
                    s.num_heads, s.num_kv_heads, s.head_dim, cache.owns, self.ctx.page_size, s.window, s.scale, s.softcap,
                    split, slots)
                return linear(self.ctx, y.view(y.shape[0], s.num_heads * s.head_dim), self.w_o, keep_split=True)
        q = K.rope_append(
            qkv, self.position.tables(batch), group.lines, k_table, v_table,
            s.num_heads, s.num_kv_heads, s.head_dim, self.position.rotary_dim, write_kv=cache.owns,
            out_dtype=self.ctx.dtype,
        )
        if K.attention_mma_takes(q.dtype, s.head_dim, heads_per_kv):
            decode, tiles, split, slots, relative = batch.attention_tiles(
                heads_per_kv, s.num_kv_heads, s.window, s.head_dim,
                K.attention_prompt_kernel(s.num_heads, s.num_kv_heads, s.head_dim, self.ctx.page_size, s.softcap))
            y = K.paged_attention_mma(
                q, k_table, v_table, group.block_table, batch.row_count, tiles,
                self.ctx.page_size, s.window, s.scale, s.softcap, decode, split, slots, relative,
                pairs=getattr(batch, "pairs", None),
            )
        else:                   # the 32-bit path, and sizes the tensor-core kernel does not take
            y = K.paged_attention_rows(
                q, k_table, v_table, group.block_table, batch.row_entry, batch.row_count,
                self.ctx.page_size, s.window, s.scale, s.softcap, batch.attention_slots(s.window),
            )
        return linear(self.ctx, y.view(y.shape[0], s.num_heads * s.head_dim), self.w_o, keep_split=True)
