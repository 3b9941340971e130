"""What a model is made of, as data: one small record for each part of each layer.

A configuration class (`gemma2.Gemma2Config`) turns config.json into a `ModelSpec`; the
engine builds parts from it through `kapel_b200.parts.registry` by each record's `kind`.
Nothing here knows a model family: sizes, constants and tensor names are all fields.

Kapel keeps one struct of switches for every family (crates/kapel-models/src/config.rs:98-166);
here a layer names its own mixer, feed-forward, norms and position encoding, so two layers
of one model may differ in all of them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """y = x / sqrt(mean(x^2) + eps) * (offset + w) for kind "rms"."""

    width: int
    eps: float
    offset: float
    weight: str                      # tensor name
    kind: str = "rms"


@dataclass(frozen=True)
class PositionSpec:
    """kind "rope": rotation of the first `rotary_dim` components, pairing "half" (j, j+r/2)."""

    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0
    pairing: str = "half"


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.

    `window` None sees every key; else a query at position p sees keys j with p - j < window.
    `scale` multiplies q.k; `softcap` c turns a score s into c*tanh(s/c) before the mask.
    `weights` maps the roles q, k, v, o to tensor names, each [out, in].
    """

    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    position: PositionSpec
    weights: Mapping[str, str]
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(h)) * up(h)); `activation` is "gelu_tanh" or "silu"."""

    hidden: int
    intermediate: int
    activation: str
    weights: Mapping[str, str]       # roles gate, up, down
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class BlockSpec:
    """The arrangement of one layer.

    kind "sandwich": norms `pre_mixer`, `post_mixer`, `pre_ffn`, `post_ffn` around both
    branches; kind "prenorm": `pre_mixer` and `pre_ffn` only.
    """

    mixer: object
    ffn: object
    norms: Mapping[str, NormSpec]
    kind: str = "sandwich"


@dataclass(frozen=True)
class ScheduleEntry:
    """One layer run: which layer, and whose cache it reads (its own when `cache_of == layer`).

    A layer named twice runs twice; a layer whose `cache_of` is another layer's index reads
    that layer's keys and values and writes none.
    """

    layer: int
    cache_of: int


@dataclass(frozen=True)
class EmbedSpec:
    weight: str
    scale: float                     # exact; rounded to the activation dtype when `round_scale`
    round_scale: bool = True
    kind: str = "embedding"


@dataclass(frozen=True)
class HeadSpec:
    weight: str                      # the table [vocab, hidden]; the embedding's when tied
    softcap: Optional[float]
    kind: str = "vocab_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embed: EmbedSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    head: HeadSpec
    max_positions: Optional[int] = None
    extra: Mapping[str, object] = field(default_factory=dict)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Each layer once, in order, with a cache of its own."""
    return tuple(ScheduleEntry(i, i) for i in range(n_layers))
