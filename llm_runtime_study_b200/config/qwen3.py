"""Typed configuration of the Qwen3 dense decoder.

Keys, defaults and checks follow the reference (mini_llm/config.py:137-188 for
the fields, :226-296 for the checks, :357-383 for the Qwen3 class).  Every size
and constant the model uses comes from here; nothing is hard-coded elsewhere.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping

from ..errors import ConfigError
from .fields import optional, required, token_id_tuple

DTYPE_BYTES = {"float16": 2, "bfloat16": 2, "float32": 4}


@dataclass(frozen=True, slots=True)
class Qwen3Config:
    """The ``config.json`` fields of a Qwen3 dense checkpoint."""

    architectures: tuple[str, ...]
    model_type: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    hidden_act: str
    attention_bias: bool
    attention_dropout: float
    tie_word_embeddings: bool
    torch_dtype: str
    bos_token_id: int
    eos_token_ids: tuple[int, ...]

    MODEL_TYPE = "qwen3"
    ARCHITECTURE = "Qwen3ForCausalLM"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        architectures = raw.get("architectures", [])
        if not isinstance(architectures, list) or not all(
            isinstance(item, str) for item in architectures
        ):
            raise ConfigError("architectures must be a list of strings")
        if raw.get("quantization_config") is not None:
            raise ConfigError(
                "quantization_config is present: quantized checkpoints are not supported"
            )
        # The reference never reads these keys (its attention is always full and its rotary
        # angles are never rescaled, mini_llm/config.py:137-188), so honouring them is not
        # possible and ignoring them would compute something else than the file asks for:
        # a null or disabled value is accepted, anything else is refused.
        if raw.get("use_sliding_window") is True and raw.get("sliding_window") is not None:
            raise ConfigError(
                "use_sliding_window is enabled: Qwen3 dense attends to the full context in this "
                "engine, as in the reference runtime; sliding-window checkpoints are not supported"
            )
        if raw.get("rope_scaling") is not None:
            raise ConfigError(
                "rope_scaling is set: rotary angles are position * theta^(-2i/d) in this engine, as in "
                "the reference runtime; scaled rotary embeddings are not supported"
            )
        config = cls(
            architectures=tuple(architectures),
            model_type=required(raw, "model_type", str),
            vocab_size=required(raw, "vocab_size", int),
            hidden_size=required(raw, "hidden_size", int),
            intermediate_size=required(raw, "intermediate_size", int),
            num_hidden_layers=required(raw, "num_hidden_layers", int),
            num_attention_heads=required(raw, "num_attention_heads", int),
            num_key_value_heads=required(raw, "num_key_value_heads", int),
            head_dim=required(raw, "head_dim", int),
            max_position_embeddings=required(raw, "max_position_embeddings", int),
            rms_norm_eps=float(required(raw, "rms_norm_eps", (int, float))),
            rope_theta=float(required(raw, "rope_theta", (int, float))),
            hidden_act=required(raw, "hidden_act", str),
            attention_bias=raw.get("attention_bias", False),
            attention_dropout=float(optional(raw, "attention_dropout", (int, float), 0.0)),
            tie_word_embeddings=raw.get("tie_word_embeddings", False),
            torch_dtype=required(raw, "torch_dtype", str),
            bos_token_id=required(raw, "bos_token_id", int),
            eos_token_ids=token_id_tuple(raw, "eos_token_id"),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.model_type != self.MODEL_TYPE:
            raise ConfigError(
                f"unsupported model_type {self.model_type!r}; expected {self.MODEL_TYPE!r}"
            )
        if self.architectures != (self.ARCHITECTURE,):
            raise ConfigError(
                f"architecture must be {self.ARCHITECTURE}, got {self.architectures}"
            )
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        ):
            value = getattr(self, name)
            if value <= 0:
                raise ConfigError(f"{name} must be positive, got {value}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "num_attention_heads must be divisible by num_key_value_heads "
                f"for grouped-query attention, got {self.num_attention_heads} and "
                f"{self.num_key_value_heads}"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(
                f"head_dim must be even for rotary embeddings, got {self.head_dim}"
            )
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if self.rope_theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"unsupported hidden_act {self.hidden_act!r}; expected 'silu'")
        if not isinstance(self.attention_bias, bool):
            raise ConfigError("attention_bias must be boolean")
        if self.attention_dropout < 0 or self.attention_dropout >= 1:
            raise ConfigError("attention_dropout must satisfy 0 <= value < 1")
        if not isinstance(self.tie_word_embeddings, bool):
            raise ConfigError("tie_word_embeddings must be boolean")
        if self.torch_dtype not in DTYPE_BYTES:
            supported = ", ".join(sorted(DTYPE_BYTES))
            raise ConfigError(
                f"unsupported torch_dtype {self.torch_dtype!r}; expected one of: {supported}"
            )
        for name, token_id in (
            ("bos_token_id", self.bos_token_id),
            *(("eos_token_id", item) for item in self.eos_token_ids),
        ):
            if not 0 <= token_id < self.vocab_size:
                raise ConfigError(
                    f"{name} must be within vocabulary [0, {self.vocab_size}), got {token_id}"
                )

    # ------------------------------------------------------------------ derived
    @property
    def query_projection_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_projection_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def queries_per_kv_head(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def validate_context_length(self, max_seq_len: int) -> None:
        if max_seq_len <= 0:
            raise ConfigError(f"max_seq_len must be positive, got {max_seq_len}")
        if max_seq_len > self.max_position_embeddings:
            raise ConfigError(
                f"max_seq_len {max_seq_len} exceeds the model limit "
                f"{self.max_position_embeddings}"
            )

    def kv_cache_bytes(self, max_seq_len: int, *, batch_size: int = 1, dtype: str = "bfloat16") -> int:
        """layers * 2 (K and V) * batch * KV heads * positions * head_dim * bytes
        (mini_llm/config.py:325-354)."""

        self.validate_context_length(max_seq_len)
        if batch_size <= 0:
            raise ConfigError(f"batch_size must be positive, got {batch_size}")
        if dtype not in DTYPE_BYTES:
            raise ConfigError(f"unsupported cache dtype {dtype!r}")
        return (
            self.num_hidden_layers * 2 * batch_size * self.num_key_value_heads
            * max_seq_len * self.head_dim * DTYPE_BYTES[dtype]
        )

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` object that reads back to this configuration."""

        raw = asdict(self)
        raw["architectures"] = list(self.architectures)
        eos = raw.pop("eos_token_ids")
        raw["eos_token_id"] = eos[0] if len(eos) == 1 else list(eos)
        return raw
