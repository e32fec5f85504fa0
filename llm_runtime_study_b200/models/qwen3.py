"""Qwen3 dense, described as parts.

Every layer is the same pre-norm block: grouped-query attention with per-head
q/k RMS norm and rotary positions, then SwiGLU (mini_llm/model/qwen.py:18-82).
All five norms share ``rms_norm_eps`` (mini_llm/model/qwen.py:34, 44-47;
mini_llm/model/base.py:49; mini_llm/nn/attention.py:291-292).  Tensor names are
the checkpoint's own (mini_llm/checkpoint.py:277-344).
"""

from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import Architecture, register_architecture
from .description import LayerDescription, ModelDescription


def describe_qwen3(config: Qwen3Config) -> ModelDescription:
    norm = {"kind": "rms_norm", "dim": config.hidden_size, "eps": config.rms_norm_eps}
    block = {
        "kind": "pre_norm",
        "mixer_norm": norm,
        "ffn_norm": norm,
        "mixer": {
            "kind": "gqa_attention",
            "hidden_size": config.hidden_size,
            "num_heads": config.num_attention_heads,
            "num_kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim,
            "bias": config.attention_bias,
            "qk_norm": {"kind": "rms_norm", "dim": config.head_dim, "eps": config.rms_norm_eps},
            "position": {"kind": "rope", "head_dim": config.head_dim, "theta": config.rope_theta},
        },
        "feed_forward": {
            "kind": "swiglu",
            "hidden_size": config.hidden_size,
            "intermediate_size": config.intermediate_size,
        },
        "names": {
            "mixer_norm": "input_layernorm",
            "mixer": "self_attn",
            "ffn_norm": "post_attention_layernorm",
            "feed_forward": "mlp",
        },
    }
    layers = tuple(
        LayerDescription(block=block, prefix=f"model.layers.{i}") for i in range(config.num_hidden_layers)
    )
    return ModelDescription(
        architecture=Qwen3Config.ARCHITECTURE,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_positions=config.max_position_embeddings,
        eos_token_ids=config.eos_token_ids,
        embedding={"prefix": "model.embed_tokens", "vocab_size": config.vocab_size, "hidden_size": config.hidden_size},
        layers=layers,
        order=tuple(range(config.num_hidden_layers)),
        final_norm={"prefix": "model.norm", **norm},
        head={
            "prefix": "lm_head", "vocab_size": config.vocab_size, "hidden_size": config.hidden_size,
            "tied": config.tie_word_embeddings,
        },
    )


QWEN3 = Architecture(
    name=Qwen3Config.ARCHITECTURE,
    model_type=Qwen3Config.MODEL_TYPE,
    config_from_dict=Qwen3Config.from_dict,
    describe=describe_qwen3,
)
register_architecture(QWEN3, replace=True)
