"""Optional text front end: a ``tokenizer.json`` beside the weights and the Qwen3
chat framing.  The engine proper starts at token ids; this module is only used
when a prompt is given as text.

Chat framing (mini_llm/chat.py:87-112): every message becomes
``<|im_start|>{role}\\n{content}<|im_end|>\\n``, then ``<|im_start|>assistant\\n``;
with thinking off an empty ``<think>\\n\\n</think>\\n\\n`` block follows.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Sequence


class TokenizerError(ValueError):
    """The tokenizer files are missing or unusable."""


@dataclass(frozen=True)
class ChatMessage:
    role: str
    content: str


def format_qwen3_chat(messages: Sequence[ChatMessage], *, enable_thinking: bool = False) -> str:
    if not messages:
        raise TokenizerError("a conversation needs at least one message")
    for m in messages:
        if m.role not in ("system", "user", "assistant"):
            raise TokenizerError(f"unknown chat role {m.role!r}")
    text = "".join(f"<|im_start|>{m.role}\n{m.content}<|im_end|>\n" for m in messages)
    text += "<|im_start|>assistant\n"
    if not enable_thinking:
        text += "<think>\n\n</think>\n\n"
    return text


class TextTokenizer:
    def __init__(self, tokenizer: Any) -> None:
        self._tokenizer = tokenizer

    def encode(self, text: str) -> list[int]:
        return list(self._tokenizer.encode(text, add_special_tokens=False).ids)

    def decode(self, token_ids: Sequence[int]) -> str:
        return self._tokenizer.decode(list(token_ids), skip_special_tokens=True)

    def encode_prompt(self, prompt: Any, *, enable_thinking: bool = False) -> list[int]:
        """A string is one user message; a list of ``ChatMessage`` (or dicts with
        ``role`` and ``content``) is a conversation."""

        if isinstance(prompt, str):
            messages = [ChatMessage("user", prompt)]
        else:
            messages = [m if isinstance(m, ChatMessage) else ChatMessage(m["role"], m["content"]) for m in prompt]
        return self.encode(format_qwen3_chat(messages, enable_thinking=enable_thinking))


def load_tokenizer(model_dir: str | Path) -> TextTokenizer:
    path = Path(model_dir) / "tokenizer.json"
    if not path.is_file():
        raise TokenizerError(f"tokenizer file does not exist: {path}")
    try:
        from tokenizers import Tokenizer
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise TokenizerError("the 'tokenizers' package is needed for text prompts") from exc
    return TextTokenizer(Tokenizer.from_file(str(path)))
