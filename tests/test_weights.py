"""Weights: the safetensors container, load errors, random weights (CPU)."""
import json
import os
import struct

import pytest
import torch

from llm_rs_b200.config import Qwen3Config
from llm_rs_b200.models.qwen3 import build_spec
from llm_rs_b200.parts import DecoderModel
from llm_rs_b200.weights import (SafetensorsFile, WeightError, WeightFileError, load_weights, open_model_files,
                                 random_tensors, save_file, write_random_model)
from tiny_configs import TINY_A, TINY_B, write_tiny_model


def _specs(raw):
    return DecoderModel(build_spec(Qwen3Config.from_dict(raw))).weight_specs()


def test_container_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file as st_save
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
               "d": torch.randn(2, 2).to(torch.float16)}
    save_file(tensors, str(tmp_path / "ours.safetensors"))
    theirs = load_file(str(tmp_path / "ours.safetensors"))
    for k, v in tensors.items():
        assert theirs[k].dtype == v.dtype and torch.equal(theirs[k], v)
    st_save(tensors, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(str(tmp_path / "theirs.safetensors"))
    assert sorted(f.names()) == sorted(tensors)
    for k, v in tensors.items():
        assert f.dtype(k) == v.dtype and f.shape(k) == tuple(v.shape) and torch.equal(f.tensor(k), v)


def test_file_errors(tmp_path):
    with pytest.raises(WeightFileError, match="no safetensors files found"):
        open_model_files(str(tmp_path))
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(WeightFileError, match="unsupported dtype"):
        SafetensorsFile(str(p))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    specs = _specs(TINY_A)
    tensors = random_tensors(specs, seed=0)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 63, dtype=torch.bfloat16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["lm_head.weight"] = torch.zeros(256, 60)   # a stored copy of the tied head: accepted, shape checked
    tensors["model.layers.0.input_layernorm.weight"] = torch.ones(64, dtype=torch.int32)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_weights(str(tmp_path), specs, torch.bfloat16, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert sorted(err.wrong_shape) == [("lm_head.weight", (256, 64), (256, 60)),
                                       ("model.layers.0.self_attn.q_proj.weight", (64, 64), (64, 63))]
    assert err.wrong_dtype == [("model.layers.0.input_layernorm.weight", "int32")]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "is [64, 63], expected [64, 64]", "model.norm.weight"):
        assert needle in text


def test_tied_model_that_also_stores_its_head(tmp_path):
    """Tied checkpoints may store ``lm_head.weight`` beside the embedding table (the reference uses a
    stored head when there is one and falls back to the table otherwise,
    llm-core/src/backends/weights.rs:143-157). Such a folder loads; the copy is not read."""
    specs = _specs(TINY_A)
    tensors = random_tensors(specs, seed=0)
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    save_file(tensors, str(tmp_path / "model.safetensors"))
    got = load_weights(str(tmp_path), specs, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in got and "model.embed_tokens.weight" in got
    model = DecoderModel(build_spec(Qwen3Config.from_dict(TINY_A)))
    from llm_rs_b200.parts import Runtime
    model.bind(got, Runtime(torch.device("cpu"), torch.bfloat16, 64))
    assert model.lm_head.proj.weight.data_ptr() == model.embedding.table.data_ptr()


def test_duplicate_across_shards(tmp_path):
    specs = _specs(TINY_A)
    tensors = random_tensors(specs, seed=0)
    save_file(tensors, str(tmp_path / "model-00001.safetensors"))
    save_file({"model.norm.weight": tensors["model.norm.weight"]}, str(tmp_path / "model-00002.safetensors"))
    with pytest.raises(WeightError, match="stored twice: model.norm.weight"):
        load_weights(str(tmp_path), specs, torch.bfloat16, "cpu")


def test_storage_rule(tmp_path):
    """bfloat16 stays bfloat16; what is stored in 32-bit stays 32-bit; norms are float32; float16 is widened."""
    specs = _specs(TINY_B)
    tensors = random_tensors(specs, seed=1)
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].float()
    tensors["model.layers.1.mlp.down_proj.weight"] = tensors["model.layers.1.mlp.down_proj.weight"].to(torch.float16)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    got = load_weights(str(tmp_path), specs, torch.bfloat16, "cpu")
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.float32
    assert got["model.layers.1.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert got["model.norm.weight"].dtype == torch.float32
    assert torch.equal(got["model.norm.weight"], tensors["model.norm.weight"].float())
    got32 = load_weights(str(tmp_path), specs, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in got32.values())
    assert torch.equal(got32["lm_head.weight"], tensors["lm_head.weight"].float())


def test_random_model_folder_is_deterministic_and_complete(tmp_path):
    a = write_tiny_model("A", str(tmp_path / "x"))
    b = write_tiny_model("A", str(tmp_path / "y"))
    fa, fb = open_model_files(a)[0], open_model_files(b)[0]
    assert sorted(fa.names()) == sorted(s.name for s in _specs(TINY_A) if s.load)
    assert "lm_head.weight" not in fa.names()       # tied
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["hidden_size"] == 64
    w = fa.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002
    n = fa.tensor("model.norm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    other = write_random_model(str(tmp_path / "z"), Qwen3Config.from_dict(TINY_A), seed=9)
    assert not torch.equal(open_model_files(other)[0].tensor("model.embed_tokens.weight"),
                           fa.tensor("model.embed_tokens.weight"))
