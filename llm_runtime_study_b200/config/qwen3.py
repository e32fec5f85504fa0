"""Typed configuration of the Qwen3 dense decoder.

Keys, defaults and checks follow the reference (mini_llm/config.py:137-188 for
the fields, :226-296 for the checks, :357-383 for the Qwen3 class).  Every size
and constant the model uses comes from here; nothing is hard-coded elsewhere.

The class itself only holds the values.  What is read and what is checked is
written down as three tables at the end of this file (``KEYS``, ``REFUSED``,
``RULES``), which ``from_dict`` and ``validate`` walk through.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Callable, Mapping

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
        """Read the keys listed in ``KEYS`` (presence and JSON type), refuse what ``REFUSED`` names,
        then apply ``RULES`` in their order; the first rule that fails raises ``ConfigError``."""

        for refuses, complaint in REFUSED:
            if refuses(raw):
                raise ConfigError(complaint)
        values = {key.field: key.read(raw) for key in KEYS}
        config = cls(**values)
        config.validate()
        return config

    def validate(self) -> None:
        for holds, complaint in RULES:
            if not holds(self):
                raise ConfigError(complaint(self))

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


# ------------------------------------------------------------------------------- the key table
# One row per config.json key the model reads (the reference's fields: mini_llm/config.py:137-188 and
# :361-367 for the key that Qwen3 adds, head_dim).  ``kinds`` is the JSON type (a bool never passes
# for an int), ``default`` is ``REQUIRED`` for keys that must be present.
REQUIRED = object()
SIZE_KEYS = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "head_dim", "max_position_embeddings")


@dataclass(frozen=True)
class Key:
    name: str
    kinds: Any
    default: Any = REQUIRED
    field: str = ""                      # attribute of Qwen3Config, when it is not the key's name
    convert: Callable[[Any], Any] = staticmethod(lambda value: value)

    def __post_init__(self) -> None:
        if not self.field:
            object.__setattr__(self, "field", self.name)

    def read(self, raw: Mapping[str, Any]) -> Any:
        if self.kinds is None:                       # the key has a reader of its own
            return self.convert(raw)
        if self.default is REQUIRED:
            return self.convert(required(raw, self.name, self.kinds))
        return self.convert(optional(raw, self.name, self.kinds, self.default))


def _architectures(raw: Mapping[str, Any]) -> tuple[str, ...]:
    listed = raw.get("architectures", [])
    if not isinstance(listed, list) or not all(isinstance(item, str) for item in listed):
        raise ConfigError("architectures must be a list of strings")
    return tuple(listed)


KEYS: tuple[Key, ...] = (
    Key("architectures", None, convert=_architectures),
    Key("model_type", str),
    *(Key(name, int) for name in SIZE_KEYS),
    Key("rms_norm_eps", (int, float), convert=float),
    Key("rope_theta", (int, float), convert=float),
    Key("hidden_act", str),
    # the two switches are type-checked by the rules below, so that their complaint names them
    Key("attention_bias", None, convert=lambda raw: raw.get("attention_bias", False)),
    Key("attention_dropout", (int, float), default=0.0, convert=float),
    Key("tie_word_embeddings", None, convert=lambda raw: raw.get("tie_word_embeddings", False)),
    Key("torch_dtype", str),
    Key("bos_token_id", int),
    Key("eos_token_id", None, field="eos_token_ids", convert=lambda raw: token_id_tuple(raw, "eos_token_id")),
)

# Keys that the reference never reads (its attention is always full and its rotary angles are never
# rescaled, mini_llm/config.py:137-188).  Honouring them is not possible and ignoring them would compute
# something else than the file asks for: a null or disabled value passes, anything else is refused.
REFUSED: tuple[tuple[Callable[[Mapping[str, Any]], bool], str], ...] = (
    (lambda raw: raw.get("quantization_config") is not None,
     "quantization_config is present: quantized checkpoints are not supported"),
    (lambda raw: raw.get("use_sliding_window") is True and raw.get("sliding_window") is not None,
     "use_sliding_window is enabled: Qwen3 dense attends to the full context in this engine, as in the "
     "reference runtime; sliding-window checkpoints are not supported"),
    (lambda raw: raw.get("rope_scaling") is not None,
     "rope_scaling is set: rotary angles are position * theta^(-2i/d) in this engine, as in the reference "
     "runtime; scaled rotary embeddings are not supported"),
)


def _positive(name: str):
    return (lambda c: getattr(c, name) > 0, lambda c: f"{name} must be positive, got {getattr(c, name)}")


def _in_vocabulary(c: "Qwen3Config") -> tuple[str, int] | None:
    """The first special token id outside ``[0, vocab_size)``, if any."""

    for name, token in (("bos_token_id", c.bos_token_id), *(("eos_token_id", t) for t in c.eos_token_ids)):
        if not 0 <= token < c.vocab_size:
            return name, token
    return None


# What must hold between the values (the reference's checks, mini_llm/config.py:235-296, one row each):
# (condition that must hold, complaint when it does not).
RULES: tuple[tuple[Callable[["Qwen3Config"], bool], Callable[["Qwen3Config"], str]], ...] = (
    (lambda c: c.model_type == c.MODEL_TYPE,
     lambda c: f"unsupported model_type {c.model_type!r}; expected {c.MODEL_TYPE!r}"),
    (lambda c: c.architectures == (c.ARCHITECTURE,),
     lambda c: f"architecture must be {c.ARCHITECTURE}, got {c.architectures}"),
    *(_positive(name) for name in SIZE_KEYS),
    (lambda c: c.num_attention_heads % c.num_key_value_heads == 0,
     lambda c: "num_attention_heads must be divisible by num_key_value_heads for grouped-query attention, "
               f"got {c.num_attention_heads} and {c.num_key_value_heads}"),
    (lambda c: c.head_dim % 2 == 0, lambda c: f"head_dim must be even for rotary embeddings, got {c.head_dim}"),
    _positive("rms_norm_eps"),
    _positive("rope_theta"),
    (lambda c: c.hidden_act == "silu", lambda c: f"unsupported hidden_act {c.hidden_act!r}; expected 'silu'"),
    (lambda c: isinstance(c.attention_bias, bool), lambda c: "attention_bias must be boolean"),
    (lambda c: 0 <= c.attention_dropout < 1, lambda c: "attention_dropout must satisfy 0 <= value < 1"),
    (lambda c: isinstance(c.tie_word_embeddings, bool), lambda c: "tie_word_embeddings must be boolean"),
    (lambda c: c.torch_dtype in DTYPE_BYTES,
     lambda c: f"unsupported torch_dtype {c.torch_dtype!r}; expected one of: {', '.join(sorted(DTYPE_BYTES))}"),
    (lambda c: _in_vocabulary(c) is None,
     lambda c: "{} must be within vocabulary [0, {}), got {}".format(_in_vocabulary(c)[0], c.vocab_size, _in_vocabulary(c)[1])),
)
