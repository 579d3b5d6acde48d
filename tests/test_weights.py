"""Weights: the container's error set (src/safetensors.ts, test/safetensors.test.ts), shards
(src/weight-files.ts, test/weight-files.test.ts), the one error that lists everything that does
not fit, and the random-weights mode."""
import json
import struct

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain
from sprout_lm_b200.config import parse_config
from sprout_lm_b200.models.decoder import DecoderModel
from sprout_lm_b200.weights import (Checkpoint, SafetensorsError, SafetensorsFile, WeightError, write_random_model,
                                    write_safetensors)


def write_raw(path, header: dict, data: bytes):
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + data)


def test_round_trip_of_the_three_dtypes(tmp_path):
    values = torch.tensor([0.0, -0.0, 1.5, -2.25, 3.0e-41, 65504.0, -1e-8, float("inf")])
    tensors = {"f32": values.clone(), "bf16": values.to(torch.bfloat16), "f16": values.to(torch.float16).reshape(2, 4)}
    write_safetensors(tmp_path / "x.safetensors", tensors, metadata={"note": "test"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    for name, tensor in tensors.items():
        got = f.tensor(name)
        assert got.dtype == tensor.dtype and got.shape == tensor.shape
        assert torch.equal(got.view(torch.int16 if got.element_size() == 2 else torch.int32),
                           tensor.view(torch.int16 if tensor.element_size() == 2 else torch.int32))
    # the plain implementation's own reader agrees (bf16 widened by a 16-bit shift)
    again = plain.read_safetensors(tmp_path / "x.safetensors")
    np.testing.assert_array_equal(again["bf16"], tensors["bf16"].float().numpy())


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "m.safetensors"
    p.write_bytes(b"\x01\x00")
    with pytest.raises(SafetensorsError, match="Truncated"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    entry = lambda dtype, shape, a, b: {"dtype": dtype, "shape": shape, "data_offsets": [a, b]}
    write_raw(p, {"t": entry("I8", [4], 0, 4)}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="Unsupported or malformed"):
        SafetensorsFile(p)
    write_raw(p, {"t": entry("F32", [2], 0, 4)}, b"\0" * 4)
    with pytest.raises(SafetensorsError, match="Invalid tensor offsets"):
        SafetensorsFile(p)
    write_raw(p, {"t": entry("F32", [2], 0, 8)}, b"\0" * 4)                       # beyond the file
    with pytest.raises(SafetensorsError, match="Invalid tensor offsets"):
        SafetensorsFile(p)
    write_raw(p, {"a": entry("F32", [1], 0, 4), "b": entry("F32", [1], 2, 6)}, b"\0" * 8)
    with pytest.raises(SafetensorsError, match="gaps or overlapping"):
        SafetensorsFile(p)
    write_raw(p, {"a": entry("F32", [1], 0, 4)}, b"\0" * 8)                       # trailing bytes
    with pytest.raises(SafetensorsError, match="does not match"):
        SafetensorsFile(p)
    write_raw(p, {"a": entry("F32", [0], 0, 0)}, b"")
    with pytest.raises(SafetensorsError, match="Unsupported or malformed"):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = parse_config(helpers.raw_config(helpers.TINY_B))
    folder = write_random_model(tmp_path / "m", config, seed=3)
    expected = {d.name: d.shape for d in DecoderModel(config.model_spec()).tensor_decls()}
    with Checkpoint(folder) as ck:
        ck.check(expected)
        tensors = {name: ck.tensor(name) for name in expected}
    del tensors["model.layers.1.self_attn.k_proj.bias"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.mlp.extra.weight"] = torch.zeros(3)
    tensors["model.layers.2.mlp.down_proj.weight"] = torch.zeros(96, 321, dtype=torch.bfloat16)
    write_safetensors(folder / "model.safetensors", tensors)
    with Checkpoint(folder) as ck, pytest.raises(WeightError) as caught:
        ck.check(expected)
    error = caught.value
    assert set(error.missing) == {"model.layers.1.self_attn.k_proj.bias", "model.norm.weight"}
    assert error.unexpected == ("model.layers.0.mlp.extra.weight",)
    assert error.wrong_shape == ("model.layers.2.mlp.down_proj.weight",)
    text = str(error)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "expected [96, 320], got [96, 321]"):
        assert piece in text


def test_tied_head_ignores_a_stray_lm_head(tmp_path):
    config = parse_config(helpers.raw_config(helpers.TINY_A))
    folder = write_random_model(tmp_path / "m", config, seed=0)
    spec = config.model_spec()
    expected = {d.name: d.shape for d in DecoderModel(spec).tensor_decls()}
    assert "lm_head.weight" not in expected
    with Checkpoint(folder) as ck:
        tensors = {name: ck.tensor(name) for name in expected}
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(folder / "model.safetensors", tensors)
    with Checkpoint(folder) as ck:
        ck.check(expected, ignorable=spec.ignorable_tensors)
        with pytest.raises(WeightError):
            ck.check(expected)


def test_sharded_folder_reads_like_a_single_file(tmp_path):
    config = parse_config(helpers.raw_config(helpers.TINY_A))
    folder = write_random_model(tmp_path / "m", config, seed=0)
    with Checkpoint(folder) as ck:
        tensors = {name: ck.tensor(name) for name in ck.inventory()}
    names = sorted(tensors)
    halves = {"part-1.safetensors": names[::2], "part-2.safetensors": names[1::2]}
    sharded = tmp_path / "sharded"
    sharded.mkdir()
    weight_map = {}
    for shard, members in halves.items():
        write_safetensors(sharded / shard, {n: tensors[n] for n in members})
        weight_map.update({n: shard for n in members})
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with Checkpoint(sharded) as ck:
        assert set(ck.inventory()) == set(names)
        for n in names:
            assert torch.equal(ck.tensor(n).float(), tensors[n].float())
        with pytest.raises(WeightError, match="Missing tensor in shard index"):
            ck.tensor("nope")
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../evil.safetensors"}}))
    with pytest.raises(WeightError, match="shard filename"):
        Checkpoint(sharded)
    (sharded / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(WeightError, match="weight map"):
        Checkpoint(sharded)


def test_random_mode_is_seeded_and_order_independent(tmp_path):
    config = parse_config(helpers.raw_config(helpers.TINY_A))
    a = write_random_model(tmp_path / "a", config, seed=7)
    b = write_random_model(tmp_path / "b", config, seed=7)
    c = write_random_model(tmp_path / "c", config, seed=8)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    assert parse_config(json.loads((a / "config.json").read_text())) == config
    _, w = plain.read_model_folder(a)
    gains = w["model.layers.0.input_layernorm.weight"]
    assert abs(float(gains.mean()) - 1.0) < 0.02 and 0.005 < float(gains.std()) < 0.04
    matrix = w["model.layers.1.mlp.gate_proj.weight"]
    assert matrix.shape == (128, 64) and abs(float(matrix.std()) - 0.02) < 0.002
    with Checkpoint(a) as ck:
        inv = ck.inventory()
        assert inv["model.embed_tokens.weight"][1] == torch.bfloat16          # matrices in bfloat16
        assert inv["model.norm.weight"][1] == torch.float32                  # 32-bit tensors stay 32-bit
        assert inv["model.layers.0.self_attn.q_proj.bias"][1] == torch.float32
