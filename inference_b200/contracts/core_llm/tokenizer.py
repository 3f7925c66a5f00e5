"""Tokenizer over the Hugging Face `tokenizers` runtime (core-llm/src/tokenizer.rs:15-88), plus the
per-token decode table the JSON constraint masks are built from."""
from __future__ import annotations

from pathlib import Path

from ..errors import InferenceError, LoadError
from .constraint import ConstraintDecodeTable


class Tokenizer:
    def __init__(self, inner):
        self.inner = inner

    @staticmethod
    def from_file(path: str | Path) -> "Tokenizer":
        import tokenizers

        try:
            return Tokenizer(tokenizers.Tokenizer.from_file(str(path)))
        except Exception as e:
            raise LoadError(f"tokenizer {path}: {e}") from e

    @staticmethod
    def from_json(text: str) -> "Tokenizer":
        import tokenizers

        try:
            return Tokenizer(tokenizers.Tokenizer.from_str(text))
        except Exception as e:
            raise LoadError(f"tokenizer json: {e}") from e

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        try:
            return list(self.inner.encode(text, add_special_tokens=add_special_tokens).ids)
        except Exception as e:
            raise InferenceError(f"encode: {e}") from e

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        try:
            return self.inner.decode(list(ids), skip_special_tokens=skip_special_tokens)
        except Exception as e:
            raise InferenceError(f"decode: {e}") from e

    def vocab_size(self) -> int:
        return self.inner.get_vocab_size(with_added_tokens=True)

    def token_to_id(self, token: str) -> int | None:
        return self.inner.token_to_id(token)

    def special_ids(self) -> set[int]:
        return {i for i, t in self.inner.get_added_tokens_decoder().items() if t.special}

    def constraint_decode_table(self) -> ConstraintDecodeTable:
        special = self.special_ids()
        pieces = []
        for i in range(self.vocab_size()):
            if i in special:
                pieces.append("")
            else:
                try:
                    pieces.append(self.inner.decode([i], skip_special_tokens=False))
                except Exception:
                    pieces.append("")
        return ConstraintDecodeTable(pieces, special)
