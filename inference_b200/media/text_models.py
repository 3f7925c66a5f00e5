"""Prompt -> (T5 sequence embedding, CLIP pooled vector) for FLUX snapshots laid out like the Hugging Face repos:
`tokenizer/{vocab.json, merges.txt}` + `text_encoder/{config.json, *.safetensors}` (CLIP-L) and
`tokenizer_2/spiece.model` + `text_encoder_2/{config.json, *.safetensors}` (T5-XXL)
(parity: candle-gen-flux/src/pipeline.rs:552-620,1011-1051: T5 ids padded to 256 / 512 and every position attended,
CLIP ids padded to 77, pooled output taken at the EOS position)."""
from __future__ import annotations

import functools
import json
from pathlib import Path

import torch

from ..contracts.errors import LoadError
from ..models.text_encoders import ClipTextConfig, ClipTextEncoder, T5Config, T5Encoder
from .text_encoders import TextConditioning


@functools.lru_cache(maxsize=1)
def _bytes_to_unicode() -> dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, map(chr, cs)))


class ClipBpeTokenizer:
    """CLIP's lower-cased byte-level BPE with `</w>` word endings, <|startoftext|> / <|endoftext|> framing."""

    def __init__(self, vocab: dict[str, int], merges: list[tuple[str, str]], max_len: int = 77):
        import regex

        self.vocab, self.max_len = vocab, max_len
        self.ranks = {m: i for i, m in enumerate(merges)}
        self.bos, self.eos = vocab["<|startoftext|>"], vocab["<|endoftext|>"]
        self.pat = regex.compile(r"<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[\p{L}]+|[\p{N}]|"
                                 r"[^\s\p{L}\p{N}]+", regex.IGNORECASE)
        self.b2u = _bytes_to_unicode()

    @staticmethod
    def from_dir(d: Path, max_len: int = 77) -> "ClipBpeTokenizer":
        vocab = json.loads((d / "vocab.json").read_text(encoding="utf-8"))
        lines = (d / "merges.txt").read_text(encoding="utf-8").split("\n")
        merges = [tuple(ln.split()) for ln in lines if ln and not ln.startswith("#version") and len(ln.split()) == 2]
        return ClipBpeTokenizer(vocab, merges, max_len)

    def _bpe(self, token: str) -> list[str]:
        word = list(token[:-1]) + [token[-1] + "</w>"]
        while len(word) > 1:
            pairs = [(self.ranks.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(word, word[1:]))]
            rank, i = min(pairs)
            if rank == 1 << 30:
                break
            a, b = word[i], word[i + 1]
            out, j = [], 0
            while j < len(word):                       # merge every occurrence of the best pair
                if j + 1 < len(word) and word[j] == a and word[j + 1] == b:
                    out.append(a + b)
                    j += 2
                else:
                    out.append(word[j])
                    j += 1
            word = out
        return word

    def encode(self, text: str, pad_id: int | None = None) -> list[int]:
        """<|startoftext|> ... <|endoftext|>, padded to max_len with `pad_id` (the end token by default)."""
        text = " ".join(text.split()).strip().lower()
        ids = [self.bos]
        unk = self.vocab.get("<|endoftext|>")
        for tok in self.pat.findall(text):
            mapped = "".join(self.b2u[b] for b in tok.encode("utf-8"))
            ids += [self.vocab.get(p, unk) for p in self._bpe(mapped)]
        ids = ids[: self.max_len - 1] + [self.eos]
        return ids + [self.eos if pad_id is None else pad_id] * (self.max_len - len(ids))


class T5SentencePieceTokenizer:
    def __init__(self, model_file: Path):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=str(model_file))
        self.eos, self.pad = 1, 0

    def encode(self, text: str, max_len: int) -> list[int]:
        ids = self.sp.encode(text)[: max_len - 1] + [self.eos]
        return ids + [self.pad] * (max_len - len(ids))


def _load_component(d: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    from ..io.safetensors_io import load_dir

    cfg_file = d / "config.json"
    if not cfg_file.is_file():
        raise LoadError(f"{d}: config.json not found")
    return json.loads(cfg_file.read_text()), load_dir(d)


class T5ClipEncoders:
    def __init__(self, t5: T5Encoder, t5_tok: T5SentencePieceTokenizer, clip: ClipTextEncoder, clip_tok: ClipBpeTokenizer):
        self.t5, self.t5_tok, self.clip, self.clip_tok = t5, t5_tok, clip, clip_tok

    @staticmethod
    def from_snapshot(root: Path, backend: str, device) -> "T5ClipEncoders":
        root = Path(root)
        dtype = torch.bfloat16 if backend == "b200" else torch.float32
        ccfg, cw = _load_component(root / "text_encoder")
        tcfg, tw = _load_component(root / "text_encoder_2")
        clip_cfg = ClipTextConfig.from_json(ccfg)
        clip = ClipTextEncoder(clip_cfg, cw, device, dtype)
        t5 = T5Encoder(T5Config.from_json(tcfg), tw, device, dtype)
        return T5ClipEncoders(t5, T5SentencePieceTokenizer(root / "tokenizer_2" / "spiece.model"), clip,
                              ClipBpeTokenizer.from_dir(root / "tokenizer", clip_cfg.max_position_embeddings))

    def encode(self, prompt: str, max_len: int) -> TextConditioning:
        t5_ids = torch.tensor([self.t5_tok.encode(prompt, max_len)], dtype=torch.int64)
        clip_ids = torch.tensor([self.clip_tok.encode(prompt)], dtype=torch.int64)
        txt = self.t5.encode(t5_ids)                     # every position attended, padding included
        _, pooled = self.clip.encode(clip_ids)
        return TextConditioning(txt, pooled)
