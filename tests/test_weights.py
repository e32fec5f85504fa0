"""Safetensors reading/writing, schema validation and random weights (no GPU)."""

import json

import pytest
import torch

from llm_runtime_study_b200.config import architecture_for
from llm_runtime_study_b200.errors import CheckpointError, CheckpointValidationError
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.weights import (
    Checkpoint, random_state, read_header, read_tensors, validate_manifest, write_file, write_random_model,
)
from tests.helpers import TINY_A, TINY_B


def _schema(raw):
    arch = architecture_for(raw)
    return tensor_schema(arch.describe(arch.config_from_dict(raw)))


def test_file_round_trip_and_library_agreement(tmp_path):
    tensors = {"b.w": torch.randn(3, 5).bfloat16(), "a": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2)}
    write_file(tmp_path / "m.safetensors", tensors)
    infos = read_header(tmp_path / "m.safetensors")
    assert [i.name for i in infos] == ["a", "b.w", "c"]
    back = read_tensors(infos)
    for name, t in tensors.items():
        assert back[name].dtype == t.dtype and torch.equal(back[name], t)
    safetensors = pytest.importorskip("safetensors.torch")
    theirs = safetensors.load_file(str(tmp_path / "m.safetensors"))
    for name, t in tensors.items():
        assert torch.equal(theirs[name], t)


def test_schema_names_and_count():
    schema = _schema(TINY_A)
    assert len(schema) == 2 * 11 + 3                      # 11 per layer, embed, norm, head
    assert schema["lm_head.weight"].optional               # tied: may be absent
    assert not _schema(TINY_B)["lm_head.weight"].optional
    assert schema["model.layers.1.self_attn.q_norm.weight"].shape == (16,)
    assert _schema(TINY_B)["model.layers.0.self_attn.q_proj.weight"].shape == (192, 96)
    assert _schema(TINY_B)["model.layers.2.mlp.down_proj.weight"].shape == (96, 272)
    assert "model.layers.0.self_attn.q_proj.bias" not in schema
    assert "model.layers.0.self_attn.k_proj.bias" in _schema({**TINY_A, "attention_bias": True})


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    write_random_model(tmp_path / "a", TINY_A, 0)
    write_random_model(tmp_path / "a2", TINY_A, 0)
    write_random_model(tmp_path / "b", TINY_A, 1)
    a, a2, b = (Checkpoint.from_model_dir(tmp_path / n).get_tensors() for n in ("a", "a2", "b"))
    assert "lm_head.weight" not in a                        # tied head left out
    assert all(torch.equal(a[n], a2[n]) for n in a)
    assert not torch.equal(a["model.embed_tokens.weight"], b["model.embed_tokens.weight"])
    validate_manifest(Checkpoint.from_model_dir(tmp_path / "a"), _schema(TINY_A), architecture="qwen3")
    emb, norm = a["model.embed_tokens.weight"], a["model.layers.0.input_layernorm.weight"]
    assert abs(float(emb.std()) - 0.02) < 0.002 and abs(float(norm.mean()) - 1.0) < 0.03
    assert json.loads((tmp_path / "a" / "config.json").read_text())["head_dim"] == 16


def test_sharded_folder_equals_single_file(tmp_path):
    write_random_model(tmp_path / "one", TINY_B, 1)
    write_random_model(tmp_path / "two", TINY_B, 1, shards=2)
    assert (tmp_path / "two" / "model.safetensors.index.json").is_file()
    one = Checkpoint.from_model_dir(tmp_path / "one")
    two = Checkpoint.from_model_dir(tmp_path / "two")
    assert one.names() == two.names()
    t1, t2 = one.get_tensors(), two.get_tensors()
    assert all(torch.equal(t1[n], t2[n]) for n in t1)


def test_one_error_lists_everything(tmp_path):
    state = random_state(_schema(TINY_B), 1, dtype=torch.float32)
    del state["model.norm.weight"]
    del state["model.layers.1.mlp.up_proj.weight"]
    state["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 96)
    state["model.layers.9.extra"] = torch.zeros(1)
    state["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(32, dtype=torch.int32)
    write_file(tmp_path / "model.safetensors", state)
    with pytest.raises(CheckpointValidationError) as err:
        validate_manifest(Checkpoint.from_model_dir(tmp_path), _schema(TINY_B), architecture="qwen3")
    text = str(err.value)
    assert "missing tensors: model.layers.1.mlp.up_proj.weight, model.norm.weight" in text
    assert "unexpected tensors: model.layers.9.extra" in text
    assert "shape mismatch for model.layers.0.self_attn.q_proj.weight: expected (192, 96), got (96, 96)" in text
    assert "dtype mismatch for model.layers.0.self_attn.k_norm.weight" in text


def test_storage_type_must_be_the_configurations_unless_relaxed(tmp_path):
    """Every floating tensor stored in config.json's torch_dtype (mini_llm/checkpoint.py:290, 478-481);
    all offenders in the one error; without a torch_dtype any floating storage is taken."""

    state = random_state(_schema(TINY_A), 0, dtype=torch.bfloat16, include_optional=False)
    state["model.norm.weight"] = state["model.norm.weight"].float()
    write_file(tmp_path / "model.safetensors", state)
    checkpoint = Checkpoint.from_model_dir(tmp_path)
    validate_manifest(checkpoint, _schema(TINY_A), architecture="qwen3")
    with pytest.raises(CheckpointValidationError) as err:
        validate_manifest(checkpoint, _schema(TINY_A), architecture="qwen3", torch_dtype="bfloat16")
    assert str(err.value).count("dtype mismatch") == 1 and "model.norm.weight: expected one of BF16, got F32" in str(err.value)
    with pytest.raises(CheckpointValidationError) as err:
        validate_manifest(checkpoint, _schema(TINY_A), architecture="qwen3", torch_dtype="float32")
    assert str(err.value).count("dtype mismatch") == len(state) - 1


def test_mapped_tensors_equal_copies_and_outlive_the_checkpoint_object(tmp_path):
    write_random_model(tmp_path, TINY_B, 1, shards=2)
    checkpoint = Checkpoint.from_model_dir(tmp_path)
    copies = checkpoint.get_tensors()
    view = checkpoint.view()
    assert sorted(view.keys()) == sorted(copies)
    kept = {name: view[name] for name in copies}
    del checkpoint, view
    assert all(torch.equal(kept[name], copies[name]) and kept[name].dtype == copies[name].dtype for name in copies)
    sub = Checkpoint.from_model_dir(tmp_path).view().sub("model.layers.1.mlp")
    assert torch.equal(sub["up_proj.weight"], copies["model.layers.1.mlp.up_proj.weight"])


def test_file_errors(tmp_path):
    with pytest.raises(CheckpointError, match="neither"):
        Checkpoint.from_model_dir(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"\x01")
    with pytest.raises(CheckpointError, match="too short"):
        Checkpoint.from_model_dir(tmp_path)
    (tmp_path / "model.safetensors").write_bytes((10**9).to_bytes(8, "little") + b"{}")
    with pytest.raises(CheckpointError, match="bad header length"):
        Checkpoint.from_model_dir(tmp_path)
    (tmp_path / "model.safetensors").unlink()
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "missing.safetensors"}}))
    with pytest.raises(CheckpointError, match="shard does not exist"):
        Checkpoint.from_model_dir(tmp_path)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {}}))
    with pytest.raises(CheckpointError, match="weight_map"):
        Checkpoint.from_model_dir(tmp_path)
    with pytest.raises(CheckpointError, match="extension"):
        read_header(tmp_path / "model.safetensors.index.json")
