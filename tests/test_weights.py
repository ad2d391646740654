"""Weights: the safetensors container and its checks (src/weight/checkpoint.cpp:502-630), model
folders, the one error that lists everything wrong, storage types, and the random-weights mode."""

import json
import struct

import pytest
import torch

from tiny_configs import TINY, tiny_config
from zephyr_b200.config import WeightError
from zephyr_b200.parts import expected_weights
from zephyr_b200.weights import (Checkpoint, RandomWeights, SafetensorsFile, WeightDecl, check_store, device_dtype,
                                 load_weights, save_safetensors, write_random_model)


def write_raw(path, header: dict, data: bytes = b""):
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + data)


def test_round_trip_all_types(tmp_path):
    tensors = {
        "a.bf16": torch.randn(3, 5).to(torch.bfloat16), "b.f32": torch.randn(7), "c.i32": torch.arange(6, dtype=torch.int32),
        "d.i64": torch.arange(4), "e.f16": torch.randn(2, 2).half(), "f.u8": torch.arange(5, dtype=torch.uint8),
        "g.bool": torch.tensor([True, False]), "h.empty": torch.empty(0, 4), "i.scalar": torch.tensor(3.5),
    }
    save_safetensors(tmp_path / "x.safetensors", tensors, metadata={"format": "pt"})
    file = SafetensorsFile(tmp_path / "x.safetensors")
    assert file.metadata == {"format": "pt"}
    for name, tensor in tensors.items():
        got = file.read(name)
        assert got.dtype == tensor.dtype and got.shape == tensor.shape and torch.equal(got, tensor)
    # The independent reader of the safetensors package agrees.
    from safetensors.torch import load_file

    theirs = load_file(str(tmp_path / "x.safetensors"))
    assert all(torch.equal(theirs[name], tensor) for name, tensor in tensors.items())


@pytest.mark.parametrize("header,data,message", [
    ({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 4, "outside the file"),
    ({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8, "needs 12"),
    ({"t": {"dtype": "F8_E4M3", "shape": [2], "data_offsets": [0, 2]}}, b"\0" * 2, "unsupported dtype"),
    ({"t": {"dtype": "F32", "shape": [2]}}, b"", "lacks dtype, shape or data_offsets"),
    ({"t": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 4]}}, b"\0" * 4, "malformed"),
    ({"a": {"dtype": "U8", "shape": [4], "data_offsets": [0, 4]},
      "b": {"dtype": "U8", "shape": [4], "data_offsets": [2, 6]}}, b"\0" * 6, "overlap"),
    ({"__metadata__": {"k": 1}}, b"", "__metadata__"),
])
def test_format_errors(tmp_path, header, data, message):
    write_raw(tmp_path / "bad.safetensors", header, data)
    with pytest.raises(WeightError, match=message):
        SafetensorsFile(tmp_path / "bad.safetensors")


def test_truncated_and_garbled_files(tmp_path):
    (tmp_path / "short.safetensors").write_bytes(b"\1\2\3")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(tmp_path / "short.safetensors")
    (tmp_path / "long.safetensors").write_bytes(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(WeightError, match="exceeds the file size"):
        SafetensorsFile(tmp_path / "long.safetensors")
    (tmp_path / "dup.safetensors").write_bytes(
        struct.pack("<Q", 88) + b'{"t":{"dtype":"U8","shape":[0],"data_offsets":[0,0]},"t":{"dtype":"U8","shape":[0],"data_offsets":[0,0]}}'[:88].ljust(88))
    with pytest.raises(WeightError):
        SafetensorsFile(tmp_path / "dup.safetensors")
    with pytest.raises(WeightError, match="cannot open"):
        SafetensorsFile(tmp_path / "absent.safetensors")


def test_folder_discovery(tmp_path):
    with pytest.raises(WeightError, match="no safetensors file"):
        Checkpoint(tmp_path)
    save_safetensors(tmp_path / "model-00001-of-00002.safetensors", {"a": torch.zeros(2)})
    with pytest.raises(WeightError, match="incomplete"):
        Checkpoint(tmp_path)
    save_safetensors(tmp_path / "model-00002-of-00002.safetensors", {"b": torch.ones(3)})
    checkpoint = Checkpoint(tmp_path)
    assert sorted(checkpoint.names()) == ["a", "b"] and torch.equal(checkpoint.read("b"), torch.ones(3))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00001-of-00002.safetensors"}}))
    with pytest.raises(WeightError, match="as the index says"):
        Checkpoint(tmp_path)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../x.safetensors"}}))
    with pytest.raises(WeightError, match="invalid file"):
        Checkpoint(tmp_path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = tiny_config("B")
    folder = write_random_model(config, 1, tmp_path / "m")
    expected = expected_weights(config.to_model_spec())
    check_store(Checkpoint(folder), expected)           # the folder as written is complete
    from safetensors.torch import load_file

    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    folder = tmp_path / "broken"
    folder.mkdir()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(31, dtype=torch.bfloat16)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    tensors["extra.bias"] = torch.zeros(3)
    save_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError) as info:
        load_weights(Checkpoint(folder), expected, torch.bfloat16, "cpu")
    text = str(info.value)
    assert "missing tensors (2)" in text and "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected tensors (2)" in text and "extra.bias" in text and "rotary_emb.inv_freq" in text
    assert "wrong shapes (2)" in text and "found [5, 5], expected [192, 96]" in text and "found [31], expected [32]" in text


def test_a_tied_checkpoint_may_carry_a_head_copy(tmp_path):
    config = tiny_config("A")
    folder = write_random_model(config, 0, tmp_path / "m")
    from safetensors.torch import load_file

    tensors = {k: v.clone() for k, v in load_file(str(folder / "model.safetensors")).items()}
    folder = tmp_path / "with_head"
    folder.mkdir()
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_safetensors(folder / "model.safetensors", tensors)
    spec = config.to_model_spec()
    loaded = load_weights(Checkpoint(folder), expected_weights(spec), torch.bfloat16, "cpu", spec.ignorable_weights)
    assert "lm_head.weight" not in loaded


def test_storage_types():
    assert device_dtype(torch.bfloat16, 2, torch.bfloat16) == torch.bfloat16
    assert device_dtype(torch.float32, 2, torch.bfloat16) == torch.bfloat16      # a matrix follows the engine
    assert device_dtype(torch.float32, 1, torch.bfloat16) == torch.float32       # a 32-bit vector stays 32-bit
    assert device_dtype(torch.float16, 1, torch.bfloat16) == torch.bfloat16
    assert device_dtype(torch.bfloat16, 1, torch.float32) == torch.float32
    assert device_dtype(torch.int64, 1, torch.bfloat16) == torch.int32

    class Store:
        data = {"w": torch.randn(4, 4), "n": torch.randn(4), "m": torch.randn(4).to(torch.bfloat16)}

        def names(self):
            return tuple(self.data)

        def shape(self, name):
            return tuple(self.data[name].shape)

        def dtype(self, name):
            return self.data[name].dtype

        def read(self, name):
            return self.data[name]

    decls = {"w": WeightDecl((4, 4)), "n": WeightDecl((4,), "norm"), "m": WeightDecl((4,), "norm")}
    out = load_weights(Store(), decls, torch.bfloat16, "cpu")
    assert (out["w"].dtype, out["n"].dtype, out["m"].dtype) == (torch.bfloat16, torch.float32, torch.bfloat16)
    out = load_weights(Store(), decls, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in out.values())
    with pytest.raises(WeightError, match="float32 or bfloat16"):
        load_weights(Store(), decls, torch.float16, "cpu")


def test_random_weights_are_seeded_per_tensor(tmp_path):
    config = tiny_config("A")
    decls = expected_weights(config.to_model_spec())
    a = RandomWeights(decls, 0, torch.float32)
    b = RandomWeights(dict(reversed(list(decls.items()))), 0, torch.float32)     # another order of tensors
    name = "model.layers.1.self_attn.o_proj.weight"
    assert torch.equal(a.read(name), b.read(name))
    assert not torch.equal(a.read(name), RandomWeights(decls, 1, torch.float32).read(name))
    linear, norm = a.read(name), a.read("model.layers.0.input_layernorm.weight")
    assert abs(float(linear.std()) - 0.02) < 0.002 and abs(float(linear.mean())) < 0.002
    assert abs(float(norm.mean()) - 1.0) < 0.01 and float(norm.std()) < 0.02
    folder = write_random_model(config, 0, tmp_path / "m")
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == TINY["A"]["config"]["hidden_size"]
    again = write_random_model(config, 0, tmp_path / "n")
    assert (folder / "model.safetensors").read_bytes() == (again / "model.safetensors").read_bytes()
    stored = Checkpoint(folder).read(name)
    assert stored.dtype == torch.bfloat16 and torch.equal(stored, linear.to(torch.bfloat16))
