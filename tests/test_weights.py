"""Weights by name: the file format's checks, one error for every misfit, seeded random weights."""
import json
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_dir
from kapel_b200.config import config_from_json
from kapel_b200.parts import expected_tensors
from kapel_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_tensors, random_tensors,
                                write_safetensors)


def test_round_trip_of_every_kept_dtype(tmp_path):
    tensors = {
        "a": torch.randn(3, 5).bfloat16(), "b": torch.arange(6, dtype=torch.int32).reshape(2, 3), "c": torch.randn(4),
        "d": torch.randn(2, 2).half(), "e": torch.arange(4, dtype=torch.int64), "empty": torch.zeros(0, 3),
    }
    write_safetensors(tmp_path / "x.safetensors", tensors)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert set(f.names()) == set(tensors)
    for k, t in tensors.items():
        assert f.dtype(k) == t.dtype and f.shape(k) == tuple(t.shape) and torch.equal(f.tensor(k), t)


def _file(tmp_path, header: bytes, data: bytes = b"", length=None):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", len(header) if length is None else length) + header + data)
    return p


def test_malformed_files_are_refused_with_the_reason(tmp_path):
    with pytest.raises(SafetensorsError, match="too short"):
        (tmp_path / "s.safetensors").write_bytes(b"abc")
        SafetensorsFile(tmp_path / "s.safetensors")
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFile(_file(tmp_path, b"{}", length=10 ** 12))
    with pytest.raises(SafetensorsError, match="not JSON"):
        SafetensorsFile(_file(tmp_path, b"{oops"))
    with pytest.raises(SafetensorsError, match="not a JSON object"):
        SafetensorsFile(_file(tmp_path, b"[1]"))
    h = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    with pytest.raises(SafetensorsError, match="needs 16"):
        SafetensorsFile(_file(tmp_path, h, b"\0" * 12))
    h = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}).encode()
    with pytest.raises(SafetensorsError, match="outside the data"):
        SafetensorsFile(_file(tmp_path, h, b"\0" * 8))
    h = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}).encode()
    with pytest.raises(SafetensorsError, match="does not take"):
        SafetensorsFile(_file(tmp_path, h, b"\0"))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_model_dir(TINY_A, 0, tmp_path / "m")
    config = config_from_json(TINY_A)
    expected = expected_tensors(config.to_spec())
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64).bfloat16()
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightsError) as info:
        load_tensors(folder, expected, "cpu")
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (16, 64), (32, 64))]
    text = str(e)
    assert "missing (2)" in text and "unexpected (1)" in text and "is [16, 64], expected [32, 64]" in text


def test_dtypes_kept_and_the_language_model_prefix(tmp_path):
    folder = make_model_dir(TINY_B, 1, tmp_path / "m")
    config = config_from_json(TINY_B)
    expected = expected_tensors(config.to_spec())
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {}
    for n in f.names():
        t = f.tensor(n).clone()
        if n.endswith("layernorm.weight"):
            t = t.float()                      # stored in 32-bit: stays so
        if n == "model.layers.0.mlp.down_proj.weight":
            t = t.half()                       # float16 becomes bfloat16
        tensors[n.replace("model.", "model.language_model.", 1)] = t
    write_safetensors(folder / "model.safetensors", tensors)
    loaded = load_tensors(folder, expected, "cpu")
    assert set(loaded) == set(expected)
    assert loaded["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert loaded["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_sharded_folder_through_its_index(tmp_path):
    folder = make_model_dir(TINY_A, 0, tmp_path / "m")
    f = SafetensorsFile(folder / "model.safetensors")
    names = sorted(f.names())
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for shard, ns in shards.items():
        write_safetensors(folder / shard, {n: f.tensor(n).clone() for n in ns})
        weight_map.update({n: shard for n in ns})
    (folder / "model.safetensors").unlink()
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    loaded = load_tensors(folder, expected_tensors(config_from_json(TINY_A).to_spec()), "cpu")
    assert len(loaded) == len(names)
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../evil.safetensors"}}))
    with pytest.raises(SafetensorsError, match="plain file name"):
        load_tensors(folder, {}, "cpu")


def test_random_weights_depend_on_name_and_seed_only():
    config = config_from_json(TINY_A)
    a, b, c = random_tensors(config, 0), random_tensors(config, 0), random_tensors(config, 1)
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    assert not torch.equal(a["model.layers.0.input_layernorm.weight"], a["model.layers.1.input_layernorm.weight"])
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert abs(float(a["model.embed_tokens.weight"].float().std()) - 0.02) < 0.002
    assert abs(float(torch.cat([a[n].float() for n in a if n.endswith("norm.weight")]).std()) - 0.1) < 0.02


def test_a_tensor_the_model_does_not_name_is_no_error_unless_strict(tmp_path):
    """Only the names the model reads are required (crates/kapel-models/src/model.rs:294-311 keeps
    every tensor of a checkpoint and asks for those it uses): an extra tensor is remembered, and an
    error only on request."""
    from kapel_b200.weights import open_weights

    folder = make_model_dir(TINY_A, 0, tmp_path / "m")
    expected = expected_tensors(config_from_json(TINY_A).to_spec())
    f = SafetensorsFile(folder / "model.safetensors")
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    tensors["vision_tower.patch.weight"] = torch.zeros(3, 5)
    write_safetensors(folder / "model.safetensors", tensors)
    loaded = load_tensors(folder, expected, "cpu")
    assert sorted(loaded) == sorted(expected)
    source = open_weights(folder, "cpu")
    assert source.check(expected) == ["vision_tower.patch.weight"] and source.unexpected == ["vision_tower.patch.weight"]
    with pytest.raises(WeightsError) as info:
        source.check(expected, strict=True)
    assert info.value.unexpected == ["vision_tower.patch.weight"] and not info.value.missing and not info.value.wrong_shape
    with pytest.raises(WeightsError):
        load_tensors(folder, expected, "cpu", strict=True)


def test_stacked_weights_are_copied_straight_into_their_rows(tmp_path):
    """`stack_rows` over a source that reads on demand equals the parts one below the other, in the
    kept dtype on the bfloat16 path and widened on the 32-bit path; `copy_into` refuses a wrong shape."""
    from kapel_b200.parts import BuildContext, stack_rows
    from kapel_b200.weights import open_weights

    folder = make_model_dir(TINY_B, 1, tmp_path / "m")
    source = open_weights(folder, "cpu")
    names = [f"model.layers.1.self_attn.{r}_proj.weight" for r in "qkv"]
    want = torch.cat([source.host(n) for n in names])
    for dtype in (torch.bfloat16, torch.float32):
        ctx = BuildContext(dtype=dtype, device=torch.device("cpu"))
        got = stack_rows(ctx, source, names)
        assert got.dtype == dtype and torch.equal(got.float(), want.float())
        assert torch.equal(stack_rows(ctx, {n: source[n] for n in names}, names), got)     # a plain dict of tensors too
    with pytest.raises(WeightsError):
        source.copy_into(names[0], torch.empty(3, 3))
    with pytest.raises(ValueError, match="cannot be stacked"):
        stack_rows(ctx, source, [names[0], "model.norm.weight"])


def test_widths_the_bfloat16_kernels_cannot_take_are_refused_when_the_parts_are_built():
    """hidden_size, heads x head_dim and intermediate_size are inner widths of bfloat16 products, read
    16 bytes at a time: a width that is no multiple of 8 is refused when the model is put together,
    with the key's name, not at the first step; the 32-bit path takes it."""
    from kapel_b200.parts import BuildContext, build_part

    raw = dict(TINY_A, hidden_size=68, intermediate_size=132)
    spec = config_from_json(raw).to_spec()
    bf16 = BuildContext(dtype=torch.bfloat16, device=torch.device("cpu"))
    with pytest.raises(ValueError, match=r"hidden_size = 68.*multiple of 8"):
        build_part("block", spec.layers[0], bf16)
    raw = dict(TINY_A, intermediate_size=132)
    with pytest.raises(ValueError, match=r"gated_mlp: intermediate_size = 132"):
        build_part("block", config_from_json(raw).to_spec().layers[0], bf16)
    f32 = BuildContext(dtype=torch.float32, device=torch.device("cpu"))
    build_part("block", spec.layers[0], f32)
