"""Prompt tokenizer for media text encoders (gen-core/src/tokenizer.rs:26-260): wraps a Hugging Face tokenizer with
a fixed prompt template, right truncation to `max_length`, optional padding, and an attention mask."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from pathlib import Path

from ..core_llm.constraint import ConstraintDecodeTable
from ..errors import InferenceError

_FLUX2_DEV_SYSTEM = ("You are an AI that reasons about image descriptions. You give structured responses focusing on "
                     "object relationships, object\nattribution and actions without speculation.")


class PromptTemplate(enum.Enum):
    """How a bare prompt is wrapped before tokenisation (the text encoders are instruction-tuned LLMs)."""
    NONE = "none"
    QWEN_INSTRUCT = "qwen_instruct"
    QWEN_INSTRUCT_NO_THINK = "qwen_instruct_no_think"
    QWEN_IMAGE = "qwen_image"
    FLUX2_DEV_MISTRAL = "flux2_dev_mistral"

    def render(self, prompt: str) -> str:
        if self is PromptTemplate.NONE:
            return prompt
        if self is PromptTemplate.QWEN_INSTRUCT:
            return f"<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"
        if self is PromptTemplate.QWEN_INSTRUCT_NO_THINK:
            return f"<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n"
        if self is PromptTemplate.QWEN_IMAGE:
            return ("<|im_start|>system\nDescribe the image by detailing the color, shape, size, texture, quantity, text, "
                    "spatial relationships of the objects and background:<|im_end|>\n<|im_start|>user\n"
                    f"{prompt}<|im_end|>\n<|im_start|>assistant\n")
        return f"[SYSTEM_PROMPT]{_FLUX2_DEV_SYSTEM}[/SYSTEM_PROMPT][INST]{prompt}[/INST]"


@dataclass
class TokenizerConfig:
    max_length: int
    pad_token_id: int = 0
    chat_template: PromptTemplate = PromptTemplate.NONE
    pad_to_max_length: bool = False


@dataclass
class TokenizerOutput:
    ids: list[int]
    mask: list[int]


class TextTokenizer:
    def __init__(self, inner, config: TokenizerConfig):
        self.inner, self._config = inner, config

    @classmethod
    def from_file(cls, path: str | Path, config: TokenizerConfig) -> "TextTokenizer":
        import tokenizers

        try:
            return cls(tokenizers.Tokenizer.from_file(str(path)), config)
        except Exception as e:
            raise InferenceError(f"tokenizer: {e}") from e

    @classmethod
    def from_json_str(cls, text: str, config: TokenizerConfig) -> "TextTokenizer":
        import tokenizers

        try:
            return cls(tokenizers.Tokenizer.from_str(text), config)
        except Exception as e:
            raise InferenceError(f"tokenizer: {e}") from e

    @classmethod
    def from_clip_bpe(cls, vocab: str | Path, merges: str | Path, config: TokenizerConfig) -> "TextTokenizer":
        """CLIP's vocab.json + merges.txt: byte-level BPE framed by <|startoftext|> ... <|endoftext|>."""
        import tokenizers
        from tokenizers import decoders, models, pre_tokenizers, processors

        try:
            bpe = models.BPE.from_file(str(vocab), str(merges), unk_token="<|endoftext|>")
            tok = tokenizers.Tokenizer(bpe)
            tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
            tok.decoder = decoders.ByteLevel()
            tok.post_processor = processors.TemplateProcessing(
                single="<|startoftext|> $A <|endoftext|>",
                pair="<|startoftext|> $A <|endoftext|> <|endoftext|> $B:1 <|endoftext|>:1",
                special_tokens=[("<|startoftext|>", 49406), ("<|endoftext|>", 49407)])
            return cls(tok, config)
        except Exception as e:
            raise InferenceError(f"tokenizer: {e}") from e

    def config(self) -> TokenizerConfig:
        return self._config

    def tokenize(self, prompt: str) -> TokenizerOutput:
        if not prompt and not self._config.pad_to_max_length:
            return TokenizerOutput([], [])
        return self.tokenize_preformatted(self._config.chat_template.render(prompt))

    def tokenize_preformatted(self, text: str) -> TokenizerOutput:
        c = self._config
        if not text and not c.pad_to_max_length:
            return TokenizerOutput([], [])
        ids = list(self.inner.encode(text, add_special_tokens=True).ids)[: c.max_length]     # right truncation
        mask = [1] * len(ids)
        if c.pad_to_max_length and len(ids) < c.max_length:
            pad = c.max_length - len(ids)
            ids += [c.pad_token_id] * pad
            mask += [0] * pad
        return TokenizerOutput(ids, mask)

    def encode_ids(self, text: str, add_special_tokens: bool) -> list[int]:
        return list(self.inner.encode(text, add_special_tokens=add_special_tokens).ids)

    def encode_chat_ids(self, prompt: str, add_special_tokens: bool) -> list[int]:
        return self.encode_ids(self._config.chat_template.render(prompt), add_special_tokens)

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return self.inner.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def constraint_decode_table(self) -> ConstraintDecodeTable:
        from ..core_llm.tokenizer import Tokenizer

        return Tokenizer(self.inner).constraint_decode_table()
