"""Prompt conditioning for FLUX-family pipelines: a sequence embedding [1, L, 4096] (T5-XXL role) and a pooled
vector [1, 768] (CLIP-L role) (parity: candle-gen-flux/src/pipeline.rs:552-620).

`HashTextEncoders` is the weight-free stand-in used by synthetic snapshots, tests and benchmarks: every byte-pair
of the prompt indexes a fixed pseudo-random table, so equal prompts give equal conditioning and different prompts
differ, with the exact shapes, dtype and padding length of the real encoders."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Protocol

import torch


@dataclass
class TextConditioning:
    txt: torch.Tensor      # [1, L, context_dim]
    pooled: torch.Tensor   # [1, vec_dim]


class TextEncoders(Protocol):
    def encode(self, prompt: str, max_len: int) -> TextConditioning: ...


class HashTextEncoders:
    def __init__(self, context_dim: int = 4096, vec_dim: int = 768, device="cpu", dtype=torch.float32):
        self.context_dim, self.vec_dim, self.device, self.dtype = context_dim, vec_dim, device, dtype

    def _vec(self, key: bytes, n: int) -> torch.Tensor:
        seed = int.from_bytes(hashlib.sha256(key).digest()[:8], "little") & 0x7FFFFFFFFFFFFFFF
        return torch.randn(n, generator=torch.Generator().manual_seed(seed), dtype=torch.float32)

    def encode(self, prompt: str, max_len: int) -> TextConditioning:
        data = prompt.encode("utf-8")
        rows = []
        for i in range(max_len):
            if i < len(data):
                rows.append(self._vec(b"tok" + data[i:i + 2] + i.to_bytes(4, "little"), self.context_dim) * 0.2)
            else:
                rows.append(self._vec(b"pad", self.context_dim) * 0.02)   # padded positions are attended too
        txt = torch.stack(rows)[None]
        pooled = self._vec(b"pool" + data, self.vec_dim)[None] * 0.5
        return TextConditioning(txt.to(self.device, self.dtype), pooled.to(self.device, self.dtype))
