"""Gemma 2's configuration: config.json's own keys, typed and checked, and its ModelSpec.

Kapel reads the same keys into its one struct of switches and classifies `gemma2` as a
sandwich block with (1 + w) RMS norms (crates/kapel-models/src/config.rs:265-509, :284).
Every size and constant comes from the file; the only values written here are the defaults
of keys a file leaves out.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .spec import (
    AttentionSpec,
    BlockSpec,
    EmbedSpec,
    GatedMLPSpec,
    HeadSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    default_schedule,
)


class ConfigError(ValueError):
    """config.json cannot describe a model this engine runs; the message names the key."""


# Bounds on sizes, as crates/kapel-models/src/config.rs:172-187,334-348 bounds them.
_MAX_LAYERS = 4096
_MAX_HEADS = 4096
_MAX_HIDDEN = 1 << 20
_MAX_HEAD_DIM = 1 << 14
_MAX_INTERMEDIATE = 1 << 24
_MAX_VOCAB = 1 << 24

# Names under which config files give the feed-forward's activation, and what they mean
# (crates/kapel-models/src/config.rs:208-219).
_ACTIVATIONS = {
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_new": "gelu_tanh",
    "gelu_fast": "gelu_tanh",
    "gelu_tanh": "gelu_tanh",
    "silu": "silu",
    "swish": "silu",
}


def _first(raw: dict, names, default=None):
    """The first of `names` that the file gives (crates/kapel-models/src/config.rs:190-205)."""
    for n in names:
        if raw.get(n) is not None:
            return raw[n]
    return default


def _int(raw, names, default=None, *, lo=1, hi=None, required=True):
    v = _first(raw, names, default)
    key = names[0]
    if v is None:
        if required:
            raise ConfigError(f"config.json: `{key}` is missing")
        return None
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v.is_integer():
            v = int(v)
        else:
            raise ConfigError(f"config.json: `{key}` must be an integer, got {v!r}")
    if v < lo or (hi is not None and v > hi):
        raise ConfigError(f"config.json: `{key}` = {v} is outside [{lo}, {hi}]")
    return v


def _float(raw, names, default=None, *, positive=True, required=False):
    v = _first(raw, names, default)
    key = names[0]
    if v is None:
        if required:
            raise ConfigError(f"config.json: `{key}` is missing")
        return None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: `{key}` must be a number, got {v!r}")
    v = float(v)
    if not math.isfinite(v) or (positive and v <= 0):
        raise ConfigError(f"config.json: `{key}` = {v} must be finite and positive")
    return v


@dataclass(frozen=True)
class Gemma2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    hidden_activation: str           # already mapped: "gelu_tanh" or "silu"
    rms_norm_eps: float
    rope_theta: float
    sliding_window: Optional[int]
    layer_types: Optional[Tuple[str, ...]]
    query_pre_attn_scalar: Optional[float]
    attn_logit_softcapping: Optional[float]
    final_logit_softcapping: Optional[float]
    tie_word_embeddings: bool
    max_position_embeddings: Optional[int]

    architecture = "Gemma2ForCausalLM"
    model_type = "gemma2"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, raw: dict) -> "Gemma2Config":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        hidden = _int(raw, ["hidden_size"], hi=_MAX_HIDDEN)
        heads = _int(raw, ["num_attention_heads"], hi=_MAX_HEADS)
        kv_heads = _int(raw, ["num_key_value_heads"], heads, hi=_MAX_HEADS)
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: `num_attention_heads` = {heads} is not a multiple of "
                f"`num_key_value_heads` = {kv_heads}"
            )
        head_dim = _int(raw, ["head_dim"], None, hi=_MAX_HEAD_DIM, required=False)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: `head_dim` is missing and `hidden_size` = {hidden} is not a "
                    f"multiple of `num_attention_heads` = {heads}"
                )
            head_dim = hidden // heads
        if head_dim % 2:
            raise ConfigError(f"config.json: `head_dim` = {head_dim} must be even (rotary pairs)")
        layers = _int(raw, ["num_hidden_layers"], hi=_MAX_LAYERS)
        act_name = _first(raw, ["hidden_activation", "hidden_act"], "gelu_pytorch_tanh")
        if act_name not in _ACTIVATIONS:
            raise ConfigError(f"config.json: `hidden_activation` = {act_name!r} is not known")
        window = _int(raw, ["sliding_window"], None, required=False)
        types = raw.get("layer_types")
        if types is not None:
            if not isinstance(types, list) or len(types) != layers:
                raise ConfigError(
                    f"config.json: `layer_types` must list {layers} layers, got "
                    f"{len(types) if isinstance(types, list) else types!r}"
                )
            for t in types:
                if t not in ("sliding_attention", "full_attention"):
                    raise ConfigError(f"config.json: `layer_types` holds {t!r}")
            if window is None and "sliding_attention" in types:
                raise ConfigError("config.json: a layer slides but `sliding_window` is missing")
            types = tuple(types)
        tie = raw.get("tie_word_embeddings", True)
        if not isinstance(tie, bool):
            raise ConfigError("config.json: `tie_word_embeddings` must be true or false")
        return cls(
            vocab_size=_int(raw, ["vocab_size"], hi=_MAX_VOCAB),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=_int(raw, ["intermediate_size"], hi=_MAX_INTERMEDIATE),
            hidden_activation=_ACTIVATIONS[act_name],
            rms_norm_eps=_float(raw, ["rms_norm_eps"], 1e-6),
            rope_theta=_float(raw, ["rope_theta"], 10000.0),
            sliding_window=window,
            layer_types=types,
            query_pre_attn_scalar=_float(raw, ["query_pre_attn_scalar"], None),
            attn_logit_softcapping=_float(raw, ["attn_logit_softcapping"], None),
            final_logit_softcapping=_float(raw, ["final_logit_softcapping"], None),
            tie_word_embeddings=tie,
            max_position_embeddings=_int(raw, ["max_position_embeddings"], None, required=False),
        )

    def to_json(self) -> dict:
        """config.json's keys again; `from_json(to_json())` is this configuration."""
        inv = {"gelu_tanh": "gelu_pytorch_tanh", "silu": "silu"}
        out = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_activation": inv[self.hidden_activation],
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
        }
        for key in (
            "sliding_window",
            "query_pre_attn_scalar",
            "attn_logit_softcapping",
            "final_logit_softcapping",
            "max_position_embeddings",
        ):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        if self.layer_types is not None:
            out["layer_types"] = list(self.layer_types)
        return out

    # ------------------------------------------------------------------ derived
    def windows(self) -> Tuple[Optional[int], ...]:
        """The window of each layer, None where a layer sees every key: `layer_types` decides;
        without it the even layers slide (crates/kapel-models/src/config.rs:349-369)."""
        out = []
        for i in range(self.num_hidden_layers):
            if self.sliding_window is None:
                out.append(None)
            elif self.layer_types is not None:
                out.append(self.sliding_window if self.layer_types[i] == "sliding_attention" else None)
            else:
                out.append(self.sliding_window if i % 2 == 0 else None)
        return tuple(out)

    def query_scale(self) -> float:
        """1/sqrt(query_pre_attn_scalar), else 1/sqrt(head_dim)
        (crates/kapel-models/src/config.rs:498; crates/kapel-ops/src/paged.rs:59-61)."""
        q = self.query_pre_attn_scalar if self.query_pre_attn_scalar is not None else self.head_dim
        return 1.0 / math.sqrt(q)

    # ------------------------------------------------------------------ the model as data
    def to_spec(self) -> ModelSpec:
        h = self.hidden_size
        position = PositionSpec(kind="rope", theta=self.rope_theta, rotary_dim=self.head_dim, pairing="half")
        windows = self.windows()

        def norm(name: str) -> NormSpec:
            return NormSpec(width=h, eps=self.rms_norm_eps, offset=1.0, weight=name)

        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}"
            mixer = AttentionSpec(
                hidden=h,
                num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                scale=self.query_scale(),
                softcap=self.attn_logit_softcapping,
                window=windows[i],
                position=position,
                weights={
                    "q": f"{p}.self_attn.q_proj.weight",
                    "k": f"{p}.self_attn.k_proj.weight",
                    "v": f"{p}.self_attn.v_proj.weight",
                    "o": f"{p}.self_attn.o_proj.weight",
                },
            )
            ffn = GatedMLPSpec(
                hidden=h,
                intermediate=self.intermediate_size,
                activation=self.hidden_activation,
                weights={
                    "gate": f"{p}.mlp.gate_proj.weight",
                    "up": f"{p}.mlp.up_proj.weight",
                    "down": f"{p}.mlp.down_proj.weight",
                },
            )
            layers.append(
                BlockSpec(
                    kind="sandwich",
                    mixer=mixer,
                    ffn=ffn,
                    norms={
                        "pre_mixer": norm(f"{p}.input_layernorm.weight"),
                        "post_mixer": norm(f"{p}.post_attention_layernorm.weight"),
                        "pre_ffn": norm(f"{p}.pre_feedforward_layernorm.weight"),
                        "post_ffn": norm(f"{p}.post_feedforward_layernorm.weight"),
                    },
                )
            )
        embed_name = "model.embed_tokens.weight"
        return ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=h,
            embed=EmbedSpec(weight=embed_name, scale=math.sqrt(h), round_scale=True),
            layers=tuple(layers),
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=norm("model.norm.weight"),
            head=HeadSpec(
                weight=embed_name if self.tie_word_embeddings else "lm_head.weight",
                softcap=self.final_logit_softcapping,
            ),
            max_positions=self.max_position_embeddings,
        )

    # ------------------------------------------------------------------ random weights
    def init_std(self, name: str, shape) -> float:
        """The standard deviation of a random tensor `name`: norm weights N(0, 0.1), applied
        as (1 + w); every table N(0, 0.02)."""
        return 0.1 if len(shape) == 1 else 0.02
