"""Safetensors reading and writing, binding by name, the one error for everything
that is wrong, and the random-weights mode."""
import json
import struct

import pytest
import torch

from tiny import TINY_A, TINY_B, make_folder

from llm_b200.config import config_from_dict
from llm_b200.engine import declared_parameters, load_model
from llm_b200.errors import FormatError, WeightError
from llm_b200.weights import (SafetensorsFile, load_checkpoint, random_tensors, write_random_model,
                              write_safetensors)


def test_write_then_read_keeps_bits_and_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7),
               "c": torch.arange(6, dtype=torch.int32).view(2, 3), "empty": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "x.safetensors", tensors, {"note": "t"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == ["a", "b", "c", "empty"] and f.metadata["note"] == "t"
    for name, t in tensors.items():
        got = f.tensor(name)
        assert got.dtype == t.dtype and got.shape == t.shape
        assert torch.equal(got.view(torch.uint8) if t.numel() else got, t.view(torch.uint8) if t.numel() else t)


def test_broken_files_are_refused(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(FormatError):
        SafetensorsFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)      # data cut short
    with pytest.raises(FormatError) as error:
        SafetensorsFile(path)
    assert "outside the file" in str(error.value)
    header = json.dumps({"w": {"dtype": "F32", "shape": [5], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 16)     # shape needs 20 bytes
    with pytest.raises(FormatError):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(FormatError):
        SafetensorsFile(path)
    with pytest.raises(FormatError):
        load_checkpoint(tmp_path / "nowhere", {})


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    config = config_from_dict(dict(TINY_A))
    expected = declared_parameters(config.model_spec())
    tensors = random_tensors(expected, 0)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(64, 32).to(torch.bfloat16)
    (tmp_path / "config.json").write_text(config.to_json())
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as error:
        load_model(tmp_path, torch.float32, "cpu")
    e = error.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert e.mismatched == [("model.layers.0.self_attn.k_proj.weight", [64, 32], [32, 64])]
    text = str(e)
    for part in e.missing + e.unexpected + ["[64, 32]", "[32, 64]"]:
        assert part in text


def test_sharded_checkpoint_through_its_index(tmp_path):
    config = config_from_dict(dict(TINY_B))
    tensors = random_tensors(declared_parameters(config.model_spec()), 9)
    names = sorted(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half],
              "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for shard, members in shards.items():
        write_safetensors(tmp_path / shard, {n: tensors[n] for n in members})
        weight_map.update({n: shard for n in members})
    (tmp_path / "config.json").write_text(config.to_json())
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    model = load_model(tmp_path, torch.float32, "cpu")
    assert torch.equal(model.head, tensors["lm_head.weight"].float())
    weight_map["model.norm.weight"] = "model-00001-of-00002.safetensors"       # not in that shard
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(FormatError):
        load_model(tmp_path, torch.float32, "cpu")


def test_tied_model_declares_no_head_and_untied_does():
    a = declared_parameters(config_from_dict(dict(TINY_A)).model_spec())
    b = declared_parameters(config_from_dict(dict(TINY_B)).model_spec())
    assert "lm_head.weight" not in a and b["lm_head.weight"].shape == (384, 96)
    assert b["model.layers.2.self_attn.q_proj.bias"].shape == (96,)
    assert "model.layers.0.self_attn.q_proj.bias" not in a
    assert a["model.layers.0.mlp.gate_proj.weight"].shape == (172, 64)


def test_random_model_folder_is_seeded_and_order_independent(tmp_path):
    config = config_from_dict(dict(TINY_B))
    one = write_random_model(tmp_path / "one", config, seed=1)
    two = write_random_model(tmp_path / "two", config, seed=1)
    other = write_random_model(tmp_path / "other", config, seed=2)
    assert (one / "model.safetensors").read_bytes() == (two / "model.safetensors").read_bytes()
    assert (one / "model.safetensors").read_bytes() != (other / "model.safetensors").read_bytes()
    assert json.loads((one / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
    f = SafetensorsFile(one / "model.safetensors")
    assert f.dtype("model.embed_tokens.weight") == torch.bfloat16
    gain = f.tensor("model.norm.weight").float()
    assert abs(float(gain.mean()) - 1.0) < 0.05                      # gains are 1 + noise
    expected = declared_parameters(config.model_spec())
    alone = random_tensors({"lm_head.weight": expected["lm_head.weight"]}, 1)
    assert torch.equal(alone["lm_head.weight"], f.tensor("lm_head.weight"))


def test_the_host_generator_equals_its_plain_statement_bit_for_bit():
    import numpy as np
    import plain_random
    from llm_b200.weights.random_init import normal_, tensor_key
    for seed, name, n in ((0, "model.embed_tokens.weight", 70001), (7, "x", 33), (123456789, "lm_head.weight", 1 << 17)):
        key = tensor_key(seed, name)
        assert key == plain_random.tensor_key(seed, name)
        want = plain_random.normal(key, n, 0.0, 0.02)
        got = normal_(torch.empty(n), key, 0.0, 0.02).numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        half = normal_(torch.empty(n, dtype=torch.bfloat16), key, 1.0, 0.02)
        want_half = torch.from_numpy(plain_random.normal(key, n, 1.0, 0.02)).to(torch.bfloat16)
        assert torch.equal(half.view(torch.int16), want_half.view(torch.int16))
    z = normal_(torch.empty(400000), tensor_key(1, "z"), 0.0, 1.0)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01
    assert abs(float((z ** 4).mean()) - 3.0) < 0.1 and float(z.abs().max()) > 4.0      # normal tails


def test_a_model_made_in_memory_equals_the_folder_of_the_same_seed(tmp_path):
    from llm_b200.engine import random_model
    config = config_from_dict(dict(TINY_B))
    folder = write_random_model(tmp_path / "m", config, seed=9, std=0.05)
    loaded = load_model(folder, torch.bfloat16, "cpu")
    made = random_model(config, 9, torch.bfloat16, "cpu", std=0.05)
    assert torch.equal(loaded.embedding, made.embedding) and torch.equal(loaded.head, made.head)
    for a, b in zip(loaded.blocks, made.blocks):
        for x, y in zip(a.weights(), b.weights()):
            assert x.dtype == y.dtype and torch.equal(x, y)
    assert torch.equal(loaded.final_norm.gain, made.final_norm.gain)


def test_storage_dtypes_and_32_bit_run(tmp_path):
    folder = make_folder(tmp_path, "A", torch.float32)
    assert SafetensorsFile(folder / "model.safetensors").dtype("model.norm.weight") == torch.float32
    model = load_model(folder, torch.float32, "cpu")
    assert model.embedding.dtype == torch.float32 and model.head is model.embedding   # tied
    half = load_model(make_folder(tmp_path, "B", torch.bfloat16), torch.bfloat16, "cpu")
    assert half.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert half.blocks[0].mixer_norm.gain.dtype == torch.float32     # gains are held in 32-bit
    assert half.blocks[0].mixer.b_qkv.dtype == torch.float32
    assert half.blocks[0].mixer.w_qkv.shape == ((3 + 2) * 32, 96)
