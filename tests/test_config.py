"""Configuration reading, typing and the architecture registry (no GPU)."""

import json

import pytest

from llm_runtime_study_b200.config import Qwen3Config, architecture_for, load_config, registered_architectures
from llm_runtime_study_b200.errors import ConfigError
from tests.helpers import TINY_A, TINY_B


def test_reads_every_size_from_the_dict():
    cfg = Qwen3Config.from_dict(TINY_B)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size) == (503, 96, 272)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (6, 1, 32)
    assert cfg.query_projection_size == 192 and cfg.kv_projection_size == 32
    assert cfg.queries_per_kv_head == 6
    assert cfg.eos_token_ids == (501, 502)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6


def test_round_trip_through_to_dict():
    for raw in (TINY_A, TINY_B):
        cfg = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("key", [
    "model_type", "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
    "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
    "rms_norm_eps", "rope_theta", "hidden_act", "torch_dtype", "bos_token_id",
])
def test_missing_required_key(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        architecture_for(raw).config_from_dict(raw) if key != "model_type" else architecture_for(
            {k: v for k, v in raw.items() if k != "architectures"})


def test_bool_is_not_an_int():
    with pytest.raises(ConfigError, match="vocab_size must be int, got bool"):
        Qwen3Config.from_dict({**TINY_A, "vocab_size": True})
    with pytest.raises(ConfigError, match="hidden_size must be int, got float"):
        Qwen3Config.from_dict({**TINY_A, "hidden_size": 64.0})


@pytest.mark.parametrize("patch,match", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"eos_token_id": 999}, "eos_token_id"),
    ({"eos_token_id": []}, "eos_token_id"),
    ({"bos_token_id": -1}, "bos_token_id"),
    ({"architectures": ["LlamaForCausalLM"]}, "architecture"),
    ({"attention_bias": 1}, "attention_bias"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"attention_dropout": 1.0}, "attention_dropout"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"quantization_config": {"bits": 4}}, "quantiz"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": 128}, "sliding"),
])
def test_rejections(patch, match):
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict({**TINY_A, **patch})


def test_keys_the_engine_does_not_use_may_be_present_when_off():
    cfg = Qwen3Config.from_dict({**TINY_A, "rope_scaling": None, "use_sliding_window": False, "sliding_window": None,
                                 "max_window_layers": 2, "use_cache": True, "transformers_version": "4.51.0"})
    assert cfg.hidden_size == 64
    Qwen3Config.from_dict({**TINY_A, "use_sliding_window": False, "sliding_window": 4096})   # off: the size does not matter


def test_context_length_and_cache_bytes():
    cfg = Qwen3Config.from_dict(TINY_A)
    cfg.validate_context_length(256)
    with pytest.raises(ConfigError):
        cfg.validate_context_length(257)
    # layers * 2 * batch * kv heads * positions * head_dim * bytes
    assert cfg.kv_cache_bytes(100, batch_size=3, dtype="bfloat16") == 2 * 2 * 3 * 2 * 100 * 16 * 2


def test_registry_and_model_dir(tmp_path):
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="does not exist"):
        load_config(tmp_path / "nope")
    with pytest.raises(ConfigError, match="configuration does not exist"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="invalid JSON"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("[1]")
    with pytest.raises(ConfigError, match="must be an object"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps({**TINY_A, "model_type": "mamba"}))
    with pytest.raises(ConfigError, match="unsupported model_type"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Qwen3ForCausalLM" and cfg.vocab_size == 503


def test_description_has_no_sizes_of_its_own():
    arch = architecture_for(TINY_B)
    desc = arch.describe(arch.config_from_dict(TINY_B))
    mixer = desc.layers[0].block["mixer"]
    assert (mixer["num_heads"], mixer["num_kv_heads"], mixer["head_dim"]) == (6, 1, 32)
    assert mixer["qk_norm"]["eps"] == 1e-5 and mixer["position"]["theta"] == 1e6
    assert desc.order == (0, 1, 2) and len(desc.layers) == 3
