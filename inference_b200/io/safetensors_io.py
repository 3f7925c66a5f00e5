"""Safetensors reader / writer without external dependencies.

The file is an 8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets}} and
the raw tensor bytes. Files are memory mapped; `load_dir` walks a sharded snapshot in sorted order
(candle-llm/src/primitives/weights.rs:17-146, candle-gen/src/loader.rs:46-207) and `slice_rows` /
`slice_cols` return a tensor-parallel shard without materialising the full tensor on the host."""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator

import numpy as np
import torch

from ..contracts.errors import LoadError

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
    "F8_E5M2": (torch.float8_e5m2, 1), "U32": (torch.uint32, 4), "U16": (torch.uint16, 2),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    start: int
    end: int

    @property
    def nbytes(self) -> int:
        return self.end - self.start


class SafetensorsFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        try:
            self._f = open(self.path, "rb")
            head = self._f.read(8)
            if len(head) != 8:
                raise LoadError(f"{self.path}: truncated safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > 512 << 20:
                raise LoadError(f"{self.path}: implausible safetensors header length {n}")
            header = json.loads(self._f.read(n))
        except (OSError, json.JSONDecodeError) as e:
            raise LoadError(f"{self.path}: {e}") from e
        self._data_start = 8 + n
        self.metadata = header.pop("__metadata__", {}) or {}
        self.tensors: dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if meta["dtype"] not in _DTYPES:
                raise LoadError(f"{self.path}: tensor {name} has unsupported dtype {meta['dtype']}")
            s, e = meta["data_offsets"]
            self.tensors[name] = TensorInfo(name, _DTYPES[meta["dtype"]][0], tuple(meta["shape"]), s, e)
        size = self.path.stat().st_size
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def keys(self) -> list[str]:
        return list(self.tensors)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def _view(self, info: TensorInfo, byte_lo: int, byte_hi: int, shape: tuple[int, ...]) -> torch.Tensor:
        buf = memoryview(self._mm)[self._data_start + byte_lo: self._data_start + byte_hi]
        if byte_hi == byte_lo:
            return torch.empty(shape, dtype=info.dtype)
        t = torch.frombuffer(buf, dtype=torch.uint8).view(info.dtype)
        return t.reshape(shape)

    def get(self, name: str) -> torch.Tensor:
        """Zero-copy tensor over a private copy-on-write mapping of the file."""
        info = self.tensors[name]
        return self._view(info, info.start, info.end, info.shape)

    def slice_rows(self, name: str, rank: int, world: int) -> torch.Tensor:
        """Rows [rank * n / world, (rank + 1) * n / world) of a tensor, read without touching the rest."""
        info = self.tensors[name]
        rows = info.shape[0]
        per = rows // world
        row_bytes = info.nbytes // max(rows, 1)
        lo, hi = info.start + rank * per * row_bytes, info.start + (rank + 1) * per * row_bytes
        return self._view(info, lo, hi, (per, *info.shape[1:]))

    def slice_cols(self, name: str, rank: int, world: int) -> torch.Tensor:
        t = self.get(name)
        per = t.shape[1] // world
        return t[:, rank * per:(rank + 1) * per]

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass  # tensors still reference the mapping; the OS releases it with the last view
        self._f.close()


def save_file(tensors: dict[str, torch.Tensor], path: str | Path, metadata: dict[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise LoadError(f"cannot save dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_file(path: str | Path, dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
    """Every tensor of one .safetensors file (copied out of the mapping)."""
    f = SafetensorsFile(path)
    try:
        return {k: (f.get(k).to(dtype) if dtype is not None else f.get(k).clone()) for k in f.keys()}
    finally:
        f.close()


def shard_files(directory: str | Path) -> list[Path]:
    d = Path(directory)
    files = sorted(p for p in d.iterdir() if p.suffix == ".safetensors") if d.is_dir() else [d]
    if not files:
        raise LoadError(f"no *.safetensors under {d}")
    return files


def iter_dir(directory: str | Path) -> Iterator[tuple[str, torch.Tensor]]:
    """Yields (name, mmap-backed tensor) over every shard in sorted file order; duplicate keys are an error."""
    seen: set[str] = set()
    for p in shard_files(directory):
        f = SafetensorsFile(p)
        for k in f.keys():
            if k in seen:
                raise LoadError(f"duplicate tensor {k} in {p}")
            seen.add(k)
            yield k, f.get(k)


def load_dir(directory: str | Path, dtype: torch.dtype | None = None, prefix: str | None = None
             ) -> dict[str, torch.Tensor]:
    out = {}
    for k, t in iter_dir(directory):
        if prefix is not None and not k.startswith(prefix):
            continue
        out[k] = t.to(dtype) if dtype is not None and t.is_floating_point() else t
    return out


def header_bytes_and_count(directory: str | Path) -> tuple[int, int]:
    """(total tensor bytes, tensor count) from headers only: weights metadata without reading tensors."""
    total = count = 0
    for p in shard_files(directory):
        f = SafetensorsFile(p)
        total += sum(i.nbytes for i in f.tensors.values())
        count += len(f.tensors)
        f.close()
    return total, count
