"""Key -> tensor map for media checkpoints (candle-gen/src/weights.rs:41-193).

Floating-point tensors are coerced to the requested dtype as they are read; integer tensors (packed quantised
weights, index tables) keep theirs. A checkpoint's tensors must each live in exactly one shard: a key seen twice
while merging shards is an error that names the key and the shard. Filtered reads only materialise tensors whose
key starts with one of the given prefixes (the safetensors file is memory-mapped, so skipped tensors cost nothing)."""
from __future__ import annotations

from pathlib import Path
from typing import Iterable, Iterator

import torch

from ..contracts.errors import LoadError
from ..io.safetensors_io import SafetensorsFile

_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def coerce_float(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return t.to(dtype) if t.dtype in _FLOATS and t.dtype != dtype else t


class Weights:
    def __init__(self, tensors: dict[str, torch.Tensor]):
        self._map = dict(tensors)

    @classmethod
    def from_map(cls, tensors: dict[str, torch.Tensor]) -> "Weights":
        return cls(tensors)

    @classmethod
    def from_file(cls, path: str | Path, device: torch.device | str = "cpu", dtype: torch.dtype = torch.bfloat16,
                  prefixes: Iterable[str] | None = None) -> "Weights":
        return cls.from_files([path], device, dtype, prefixes)

    @classmethod
    def from_files(cls, files: Iterable[str | Path], device: torch.device | str = "cpu",
                   dtype: torch.dtype = torch.bfloat16, prefixes: Iterable[str] | None = None) -> "Weights":
        pref = tuple(prefixes) if prefixes is not None else None
        out: dict[str, torch.Tensor] = {}
        for path in files:
            st = SafetensorsFile(path)
            try:
                for k in st.keys():
                    if pref is not None and not k.startswith(pref):
                        continue
                    if k in out:
                        raise LoadError(
                            f"duplicate tensor key {k!r} while merging shard {path}: a checkpoint's tensors must each "
                            f"live in exactly one .safetensors shard - this snapshot has {k!r} in more than one file "
                            "(mis-sharded checkpoint or a stray .safetensors in the dir)")
                    out[k] = coerce_float(st.get(k), dtype).to(device)
            finally:
                st.close()
        return cls(out)

    def device(self) -> torch.device | None:
        for t in self._map.values():
            return t.device
        return None

    def require(self, key: str) -> torch.Tensor:
        t = self._map.get(key)
        if t is None:
            raise LoadError(f"missing tensor: {key}")
        return t

    def contains(self, key: str) -> bool:
        return key in self._map

    __contains__ = contains

    def keys(self) -> Iterator[str]:
        return iter(self._map.keys())

    def with_prefix(self, prefix: str) -> "Weights":
        """The sub-map under `prefix`, with the prefix stripped from the keys."""
        return Weights({k[len(prefix):]: v for k, v in self._map.items() if k.startswith(prefix)})

    def __len__(self) -> int:
        return len(self._map)
