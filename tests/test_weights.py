"""Weights by name: the reader and writer, the one error that lists everything, random weights (no GPU)."""

import json

import pytest
import torch

from tests.tiny_configs import TINY_A, TINY_B, tensor_shapes, tiny_weights, write_model_folder
from tokensprint_b200.models.qwen3 import Qwen3Config
from tokensprint_b200.models.qwen3 import build_qwen3_spec
from tokensprint_b200.weights.loader import (
    FolderSource,
    LoadedTensors,
    RandomSource,
    WeightsError,
    check_tensors,
    write_random_model,
)
from tokensprint_b200.weights.safetensors_io import SafetensorsError, SafetensorsFolder, save_safetensors


def test_spec_names_are_the_checkpoint_names():
    for cfg in (TINY_A, TINY_B):
        specs = build_qwen3_spec(Qwen3Config.from_dict(cfg)).tensor_specs()
        assert {s.name: tuple(s.shape) for s in specs} == tensor_shapes(cfg)
        assert {s.role for s in specs if s.name.endswith("norm.weight") or "layernorm" in s.name} == {"vector"}


def test_reader_agrees_with_the_safetensors_package(tmp_path):
    w = tiny_weights(TINY_A, 3)
    w["some.bf16"] = torch.randn(5, 7).to(torch.bfloat16)
    w["some.i32"] = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    write_model_folder(tmp_path, TINY_A, w)
    folder = SafetensorsFolder(tmp_path)
    assert sorted(folder.keys()) == sorted(w)
    for name, t in w.items():
        got = folder.tensor(name)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape)
        assert torch.equal(got, t)


def test_writer_is_read_by_the_safetensors_package(tmp_path):
    from safetensors import safe_open

    tensors = {"a": torch.randn(3, 4), "b": torch.randn(8).to(torch.bfloat16), "c": torch.tensor(3, dtype=torch.int32)}
    save_safetensors(tmp_path / "x.safetensors", tensors.items())
    with safe_open(str(tmp_path / "x.safetensors"), framework="pt") as f:
        assert sorted(f.keys()) == ["a", "b", "c"]
        for k, v in tensors.items():
            assert torch.equal(f.get_tensor(k), v)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    specs = build_qwen3_spec(cfg).tensor_specs()
    w = tiny_weights(TINY_B, 1)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(4)
    w["model.layers.2.self_attn.k_norm.weight"] = torch.zeros(7)
    w["lm_head.weight"] = torch.zeros(3, 3)
    write_model_folder(tmp_path, TINY_B, w)
    src = FolderSource(tmp_path)
    with pytest.raises(WeightsError) as e:
        check_tensors(specs, src.shapes(), where=str(tmp_path))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(err.wrong_shape) == 2
    msg = str(err)
    for word in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "k_norm.weight: expected [32], found [7]", "lm_head.weight"):
        assert word in msg


def test_stray_lm_head_beside_tied_embeddings_is_ignored(tmp_path):
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_A))
    w = tiny_weights(TINY_A, 1)
    w["lm_head.weight"] = torch.zeros(256, 64)
    write_model_folder(tmp_path, TINY_A, w)
    check_tensors(spec.tensor_specs(), FolderSource(tmp_path).shapes(), ignorable=spec.ignorable_tensors)
    with pytest.raises(WeightsError):
        check_tensors(spec.tensor_specs(), FolderSource(tmp_path).shapes())


def test_device_dtypes_by_role(tmp_path):
    spec = build_qwen3_spec(Qwen3Config.from_dict(TINY_A))
    write_model_folder(tmp_path, TINY_A, tiny_weights(TINY_A, 1), dtype=torch.bfloat16)
    specs = spec.tensor_specs()
    for compute in (torch.bfloat16, torch.float32):
        t = LoadedTensors(FolderSource(tmp_path), specs, torch.device("cpu"), compute)
        assert t["model.embed_tokens.weight"].dtype == compute
        assert t["model.layers.0.self_attn.q_norm.weight"].dtype == torch.float32
        assert t["model.norm.weight"].dtype == torch.float32


def test_bad_files_fail_loudly(tmp_path):
    with pytest.raises(FileNotFoundError):
        SafetensorsFolder(tmp_path / "nope")
    with pytest.raises(SafetensorsError, match="No safetensors files"):
        SafetensorsFolder(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!!")
    with pytest.raises(SafetensorsError):
        SafetensorsFolder(tmp_path)


def test_random_weights_mode_writes_a_model_folder(tmp_path):
    cfg = Qwen3Config.from_dict(TINY_B)
    folder = write_random_model(tmp_path / "m", cfg, seed=5, dtype="bfloat16")
    assert json.loads((folder / "config.json").read_text())["hidden_size"] == 96
    files = SafetensorsFolder(folder)
    assert {n: files.shape(n) for n in files.keys()} == tensor_shapes(TINY_B)
    assert files.dtype("lm_head.weight") == torch.bfloat16
    q = files.tensor("model.layers.1.self_attn.q_proj.weight").float()
    assert abs(q.std().item() - 0.02) < 0.002 and abs(q.mean().item()) < 0.002
    n = files.tensor("model.norm.weight").float()
    assert abs(n.mean().item() - 1.0) < 0.03
    # same seed, same values; other seed, other values; the folder equals the direct source
    again = write_random_model(tmp_path / "m2", cfg, seed=5, dtype="bfloat16")
    other = write_random_model(tmp_path / "m3", cfg, seed=6, dtype="bfloat16")
    a, b, c = (SafetensorsFolder(p).tensor("model.layers.0.mlp.down_proj.weight") for p in (folder, again, other))
    assert torch.equal(a, b) and not torch.equal(a, c)
    specs = build_qwen3_spec(cfg).tensor_specs()
    direct = LoadedTensors(RandomSource(specs, 5), specs, torch.device("cpu"), torch.bfloat16)
    assert torch.equal(direct["model.layers.0.mlp.down_proj.weight"], a)
