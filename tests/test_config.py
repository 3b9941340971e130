"""Configuration: config.json's keys, defaults, checks, the registry, the model as data."""
import json
import math

import pytest

from helpers import TINY_A, TINY_B
from kapel_b200.config import (ConfigError, Gemma2Config, config_from_dir, config_from_json, register_architecture,
                               unregister_architecture)


def test_keys_are_read_as_given():
    c = Gemma2Config.from_json(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 6, 1, 32)
    assert (c.intermediate_size, c.vocab_size, c.rope_theta, c.sliding_window) == (320, 1000, 500000.0, 24)
    assert (c.attn_logit_softcapping, c.final_logit_softcapping, c.rms_norm_eps) == (20.0, 15.0, 1e-5)
    assert c.windows() == (24, None, 24)
    assert c.query_scale() == pytest.approx(1 / math.sqrt(24))
    assert Gemma2Config.from_json(c.to_json()) == c


def test_defaults_of_missing_keys():
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "query_pre_attn_scalar", "rms_norm_eps",
                                                         "rope_theta", "hidden_activation", "attn_logit_softcapping", "final_logit_softcapping")}
    c = Gemma2Config.from_json(raw)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4
    assert c.query_scale() == pytest.approx(1 / math.sqrt(16))         # 1/sqrt(head_dim) without the key
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.hidden_activation == "gelu_tanh"
    assert c.attn_logit_softcapping is None and c.final_logit_softcapping is None
    assert c.windows() == (16, None)                                  # even layers slide without layer_types


def test_hidden_act_alias_and_layer_types():
    raw = dict(TINY_A)
    del raw["hidden_activation"]
    raw["hidden_act"] = "gelu_new"
    raw["layer_types"] = ["full_attention", "sliding_attention"]
    c = Gemma2Config.from_json(raw)
    assert c.hidden_activation == "gelu_tanh" and c.windows() == (None, 16)


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": 0}, "hidden_size"), ({"num_hidden_layers": -1}, "num_hidden_layers"),
    ({"num_attention_heads": 4, "num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
    ({"vocab_size": None}, "vocab_size"), ({"hidden_activation": "relu6"}, "hidden_activation"),
    ({"layer_types": ["sliding_attention"]}, "layer_types"), ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"intermediate_size": "big"}, "intermediate_size"), ({"num_hidden_layers": 5000}, "outside"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_bad_values_are_errors_not_crashes(change, match):
    with pytest.raises(ConfigError, match=match):
        Gemma2Config.from_json(dict(TINY_A, **change))


def test_registry_by_architecture_then_model_type(tmp_path):
    assert isinstance(config_from_json(TINY_A), Gemma2Config)
    assert isinstance(config_from_json({**TINY_A, "architectures": ["Other"]}), Gemma2Config)     # model_type decides
    with pytest.raises(ConfigError, match="unsupported architecture"):
        config_from_json({**TINY_A, "architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_dir(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        config_from_dir(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    cfg, raw = config_from_dir(tmp_path)
    assert cfg == Gemma2Config.from_json(TINY_B) and raw["vocab_size"] == 1000


def test_another_architecture_registers_without_touching_the_package():
    class Other(Gemma2Config):
        architecture = "OtherForCausalLM"

    register_architecture(Other, "OtherForCausalLM")
    try:
        assert type(config_from_json({**TINY_A, "architectures": ["OtherForCausalLM"]})) is Other
        with pytest.raises(ValueError, match="already registered"):
            register_architecture(Gemma2Config, "OtherForCausalLM")
    finally:
        unregister_architecture("OtherForCausalLM")


def test_spec_describes_every_layer_by_its_own_parts():
    spec = Gemma2Config.from_json(TINY_B).to_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert [l.mixer.window for l in spec.layers] == [24, None, 24]
    m = spec.layers[1].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.softcap) == (6, 1, 32, 20.0)
    assert m.position.theta == 500000.0 and m.position.rotary_dim == 32
    assert spec.layers[0].ffn.intermediate == 320 and spec.layers[0].ffn.activation == "gelu_tanh"
    assert set(spec.layers[0].norms) == {"pre_mixer", "post_mixer", "pre_ffn", "post_ffn"}
    assert spec.layers[2].norms["post_ffn"].eps == 1e-5 and spec.layers[2].norms["post_ffn"].offset == 1.0
    assert spec.embed.scale == pytest.approx(math.sqrt(96)) and spec.head.weight == spec.embed.weight
    assert spec.head.softcap == 15.0 and spec.max_positions == 256
    untied = Gemma2Config.from_json({**TINY_B, "tie_word_embeddings": False}).to_spec()
    assert untied.head.weight == "lm_head.weight"
