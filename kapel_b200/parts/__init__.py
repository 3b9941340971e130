"""Layer parts: mixers, feed-forwards, norms, position encodings, blocks, and the two ends."""
from .attention import Attention
from .base import BuildContext, LayerCache, Part, linear, matrix_for, matrix_named, require_product_widths, stack_rows
from .block import PreNormBlock, SandwichBlock
from .embedding import Embedding, VocabHead
from .feed_forward import GatedMLP
from .norm import RMSNorm, add_branch
from .position import NoPosition, Rope
from .registry import (
    build_part,
    part_class,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_part,
    register_position,
    unregister_part,
)

register_part("mixer", "attention", Attention)
register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("norm", "rms", RMSNorm)
register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
register_part("block", "sandwich", SandwichBlock)
register_part("block", "prenorm", PreNormBlock)
register_part("embedding", "embedding", Embedding)
register_part("head", "vocab_head", VocabHead)


def expected_tensors(spec) -> dict:
    """{tensor name: shape} of everything a model built from `spec` reads."""
    out = {spec.embed.weight: (spec.vocab_size, spec.hidden_size)}
    out[spec.head.weight] = (spec.vocab_size, spec.hidden_size)
    n = spec.final_norm
    out.update(part_class("norm", n.kind).expected_tensors(n))
    for layer in spec.layers:
        out.update(part_class("block", layer.kind).expected_tensors(layer))
    return out
