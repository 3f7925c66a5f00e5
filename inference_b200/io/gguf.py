"""GGUF container: reader (header, key/value metadata, tensor table, mmap'd data), writer, and conversion to
an HF-style checkpoint (name remap, llama q/k un-permute, config and tokenizer reconstruction).

Parity: candle-llm/src/gguf.rs:36-448 (open, gguf_architecture probe, gguf_arch_to_hf, key remap at :293-318,
q/k un-permute at :333-356); container layout per mlx-llm/src/gguf/reader.rs."""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from ..contracts.errors import LoadError, Unsupported
from . import gguf_quants as gq

MAGIC = b"GGUF"
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


@dataclass(frozen=True)
class GgufTensorInfo:
    name: str
    shape: tuple[int, ...]   # row-major (outermost first); GGUF stores dims innermost-first
    type_name: str
    offset: int              # relative to the data section
    nbytes: int


class _Reader:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def take(self, fmt: str):
        n = struct.calcsize(fmt)
        if self.pos + n > len(self.buf):
            raise LoadError("GGUF: truncated file")
        (v,) = struct.unpack_from(fmt, self.buf, self.pos)
        self.pos += n
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise LoadError("GGUF: truncated string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, t: int):
        if t in _SCALARS:
            return self.take(_SCALARS[t])
        if t == 8:
            return self.string()
        if t == 9:
            et = self.take("<I")
            n = self.take("<Q")
            if et in _SCALARS and et != 7:
                fmt = _SCALARS[et]
                size = struct.calcsize(fmt)
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=n, offset=self.pos)
                self.pos += size * n
                return arr.tolist()
            return [self.value(et) for _ in range(n)]
        raise LoadError(f"GGUF: unknown metadata value type {t}")


class GgufFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            self._f = open(self.path, "rb")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except (OSError, ValueError) as e:
            raise LoadError(f"{self.path}: {e}") from e
        r = _Reader(self._mm)
        if bytes(self._mm[:4]) != MAGIC:
            raise LoadError(f"{self.path}: not a GGUF file (bad magic)")
        r.pos = 4
        self.version = r.take("<I")
        if self.version < 2:
            raise Unsupported(f"{self.path}: GGUF version {self.version} is not supported")
        n_tensors, n_kv = r.take("<Q"), r.take("<Q")
        self.metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            k = r.string()
            self.metadata[k] = r.value(r.take("<I"))
        self.tensors: dict[str, GgufTensorInfo] = {}
        for _ in range(n_tensors):
            name = r.string()
            nd = r.take("<I")
            dims = [r.take("<Q") for _ in range(nd)]
            tname = gq.type_name(r.take("<I"))
            off = r.take("<Q")
            n_el = int(np.prod(dims)) if dims else 1
            self.tensors[name] = GgufTensorInfo(name, tuple(reversed(dims)), tname, off, gq.nbytes(tname, n_el))
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (r.pos + align - 1) // align * align

    def architecture(self) -> str | None:
        a = self.metadata.get("general.architecture")
        return a if isinstance(a, str) else None

    def raw(self, name: str) -> np.ndarray:
        i = self.tensors[name]
        return np.frombuffer(self._mm, dtype=np.uint8, count=i.nbytes, offset=self.data_start + i.offset)

    def dequantize(self, name: str) -> torch.Tensor:
        i = self.tensors[name]
        n = int(np.prod(i.shape)) if i.shape else 1
        return torch.from_numpy(gq.dequantize(self.raw(name), i.type_name, n).reshape(i.shape).copy())

    def close(self) -> None:
        try:
            self._mm.close()
        except BufferError:
            pass
        self._f.close()


def gguf_architecture(path: str | Path) -> str | None:
    """Weightless probe: reads only the header and metadata."""
    try:
        f = GgufFile(path)
    except (LoadError, Unsupported):
        return None
    a = f.architecture()
    f.close()
    return a


ARCH_TO_HF = {"llama": ("LlamaForCausalLM", "llama"), "qwen3": ("Qwen3ForCausalLM", "qwen3"),
              "qwen2": ("Qwen2ForCausalLM", "qwen2"), "mistral": ("MistralForCausalLM", "mistral")}

_LAYER_MAP = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
              "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm",
              "attn_k_norm": "self_attn.k_norm", "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj",
              "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


def hf_name(gguf_name: str) -> str | None:
    top = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
           "output.weight": "lm_head.weight"}
    if gguf_name in top:
        return top[gguf_name]
    parts = gguf_name.split(".")
    if len(parts) == 4 and parts[0] == "blk" and parts[1].isdigit() and parts[2] in _LAYER_MAP:
        return f"model.layers.{parts[1]}.{_LAYER_MAP[parts[2]]}.{parts[3]}"
    return None


def unpermute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """Inverse of the llama.cpp converter's rotary row permutation, back to the HF half-split layout."""
    rows = w.shape[0]
    return w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def permute_qk(w: torch.Tensor, n_head: int) -> torch.Tensor:
    rows = w.shape[0]
    return w.reshape(n_head, 2, rows // n_head // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


class GgufCheckpoint:
    """A GGUF file viewed as an HF checkpoint: config dict, dense tensors under HF names, tokenizer JSON."""

    def __init__(self, path: str | Path):
        self.file = GgufFile(path)
        arch = self.file.architecture()
        if arch not in ARCH_TO_HF:
            raise Unsupported(f"GGUF architecture {arch!r} is not supported (supported: {sorted(ARCH_TO_HF)})")
        self.arch = arch

    @staticmethod
    def open(path: str | Path) -> "GgufCheckpoint":
        return GgufCheckpoint(path)

    def config(self) -> dict[str, Any]:
        md, a = self.file.metadata, self.arch

        def g(key, default=None):
            return md.get(f"{a}.{key}", default)

        hidden = int(g("embedding_length"))
        heads = int(g("attention.head_count"))
        hf_arch, model_type = ARCH_TO_HF[a]
        vocab = len(md.get("tokenizer.ggml.tokens", [])) or self.file.tensors["token_embd.weight"].shape[0]
        ffn = g("feed_forward_length")
        cfg = {"architectures": [hf_arch], "model_type": model_type, "hidden_size": hidden,
               "num_hidden_layers": int(g("block_count")), "num_attention_heads": heads,
               "num_key_value_heads": int(g("attention.head_count_kv", heads)),
               "intermediate_size": int(ffn[0] if isinstance(ffn, list) else ffn), "vocab_size": int(vocab),
               "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)),
               "rope_theta": float(g("rope.freq_base", 10000.0)),
               "max_position_embeddings": int(g("context_length", 0)),
               "tie_word_embeddings": "output.weight" not in self.file.tensors}
        if g("attention.key_length") is not None:
            cfg["head_dim"] = int(g("attention.key_length"))
        for key, name in (("tokenizer.ggml.bos_token_id", "bos_token_id"), ("tokenizer.ggml.eos_token_id", "eos_token_id")):
            if key in md:
                cfg[name] = int(md[key])
        return cfg

    def tensors(self, dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
        """Every tensor dequantised to dense under its HF name (llama q/k rows un-permuted)."""
        cfg = self.config()
        out = {}
        for name in self.file.tensors:
            hf = hf_name(name)
            if hf is None:
                continue
            t = self.file.dequantize(name)
            if self.arch == "llama" and hf.endswith("self_attn.q_proj.weight"):
                t = unpermute_qk(t, cfg["num_attention_heads"])
            elif self.arch == "llama" and hf.endswith("self_attn.k_proj.weight"):
                t = unpermute_qk(t, cfg["num_key_value_heads"])
            out[hf] = t.to(dtype)
        return out

    def chat_template(self) -> str | None:
        t = self.file.metadata.get("tokenizer.chat_template")
        return t if isinstance(t, str) else None

    def tokenizer_json(self) -> str | None:
        """Rebuilds a `tokenizers` JSON for byte-level BPE vocabularies (tokenizer.ggml.model == "gpt2")."""
        md = self.file.metadata
        tokens = md.get("tokenizer.ggml.tokens")
        if not isinstance(tokens, list) or md.get("tokenizer.ggml.model") != "gpt2":
            return None
        merges = md.get("tokenizer.ggml.merges") or []
        types = md.get("tokenizer.ggml.token_type") or []
        added = [{"id": i, "content": tokens[i], "single_word": False, "lstrip": False, "rstrip": False,
                  "normalized": False, "special": True} for i, t in enumerate(types) if t == 3]
        spec = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": added, "normalizer": None,
                "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True,
                                  "use_regex": True},
                "post_processor": None,
                "decoder": {"type": "ByteLevel", "add_prefix_space": True, "trim_offsets": True, "use_regex": True},
                "model": {"type": "BPE", "dropout": None, "unk_token": None, "continuing_subword_prefix": None,
                          "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False,
                          "vocab": {t: i for i, t in enumerate(tokens)}, "merges": list(merges)}}
        return json.dumps(spec)


# ---- writer (used by snapshot tooling and tests) ----------------------------------------------------------
def _w_string(out: bytearray, s: str) -> None:
    b = s.encode()
    out += struct.pack("<Q", len(b)) + b


def _w_value(out: bytearray, v: Any) -> None:
    if isinstance(v, bool):
        out += struct.pack("<I?", 7, v)
    elif isinstance(v, int):
        out += struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<II", 4, v) if v < 2 ** 32 else struct.pack("<IQ", 10, v)
    elif isinstance(v, float):
        out += struct.pack("<If", 6, v)
    elif isinstance(v, str):
        out += struct.pack("<I", 8)
        _w_string(out, v)
    elif isinstance(v, list):
        out += struct.pack("<I", 9)
        if all(isinstance(x, str) for x in v):
            out += struct.pack("<IQ", 8, len(v))
            for x in v:
                _w_string(out, x)
        elif all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            out += struct.pack("<IQ", 5, len(v)) + np.asarray(v, dtype="<i4").tobytes()
        else:
            out += struct.pack("<IQ", 6, len(v)) + np.asarray(v, dtype="<f4").tobytes()
    else:
        raise LoadError(f"GGUF writer: unsupported metadata value {type(v)}")


def write_gguf(path: str | Path, metadata: dict[str, Any], tensors: dict[str, tuple[np.ndarray, str, tuple[int, ...]]],
               alignment: int = 32) -> None:
    """tensors: name -> (raw uint8 bytes, ggml type name, row-major shape)."""
    out = bytearray(MAGIC + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for k, v in metadata.items():
        _w_string(out, k)
        _w_value(out, v)
    offset = 0
    blobs = []
    for name, (raw, tname, shape) in tensors.items():
        _w_string(out, name)
        out += struct.pack("<I", len(shape))
        for d in reversed(shape):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", gq.TYPE_IDS[tname], offset)
        b = np.ascontiguousarray(raw).view(np.uint8).reshape(-1).tobytes()
        pad = (alignment - len(b) % alignment) % alignment
        blobs.append(b + b"\0" * pad)
        offset += len(b) + pad
    out += b"\0" * ((alignment - len(out) % alignment) % alignment)
    with open(path, "wb") as f:
        f.write(out)
        for b in blobs:
            f.write(b)
