"""Checkpoint metadata without reading tensors, and adapter key conventions (gen-core/src/weightsmeta.rs:50-591).

`CheckpointMeta` reads safetensors headers only (a file or every shard of a directory). The adapter helpers classify
LoRA / LoKr / LoHa / kohya key layouts, find the key prefix, parse rank / alpha strings defensively and map kohya
`lora_unet_a_b_c` stems back to dotted module paths."""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from pathlib import Path

from ..errors import LoadError

COMMON_LORA_PREFIXES = ("transformer.", "diffusion_model.")
KOHYA_PREFIX = "lora_unet_"
LORA_ADAPTER_METADATA_KEY = "lora_adapter_metadata"
_DTYPE_BYTES = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1,
                "F8_E4M3": 1, "F8_E5M2": 1, "U16": 2, "U32": 4, "U64": 8}


def is_hidden_file(path: Path) -> bool:
    return Path(path).name.startswith((".", "._"))


@dataclass(frozen=True)
class TensorMeta:
    dtype: str
    shape: tuple[int, ...]
    nbytes: int


@dataclass
class CheckpointMeta:
    tensors: dict[str, TensorMeta] = field(default_factory=dict)
    metadata: dict[str, str] = field(default_factory=dict)

    @staticmethod
    def _read_header(path: Path) -> dict:
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise LoadError(f"{path}: not a safetensors file (too short)")
            (n,) = struct.unpack("<Q", head)
            if n > (100 << 20):
                raise LoadError(f"{path}: implausible safetensors header of {n} bytes")
            try:
                return json.loads(f.read(n))
            except json.JSONDecodeError as e:
                raise LoadError(f"{path}: malformed safetensors header: {e}")

    @staticmethod
    def from_file(path) -> "CheckpointMeta":
        path = Path(path)
        h = CheckpointMeta._read_header(path)
        m = CheckpointMeta(metadata={str(k): str(v) for k, v in (h.pop("__metadata__", None) or {}).items()})
        for k, v in h.items():
            lo, hi = v["data_offsets"]
            m.tensors[k] = TensorMeta(v["dtype"], tuple(v["shape"]), hi - lo)
        return m

    @staticmethod
    def from_dir(d) -> "CheckpointMeta":
        files = sorted(p for p in Path(d).glob("*.safetensors") if not is_hidden_file(p))
        if not files:
            raise LoadError(f"{d}: no safetensors files")
        out = CheckpointMeta()
        for f in files:
            m = CheckpointMeta.from_file(f)
            out.tensors.update(m.tensors)
            out.metadata.update(m.metadata)
        return out

    def keys(self):
        return self.tensors.keys()

    def contains(self, key: str) -> bool:
        return key in self.tensors

    def total_bytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())


def safetensors_path_bytes(path) -> int:
    """Tensor bytes of a file or directory from headers only; 0 when nothing readable is there."""
    p = Path(path)
    try:
        return (CheckpointMeta.from_dir(p) if p.is_dir() else CheckpointMeta.from_file(p)).total_bytes()
    except (LoadError, OSError):
        return 0


def is_lokr_network_type(network_type: str | None) -> bool:
    return network_type is not None and network_type.strip().lower() == "lokr"


def keys_contain_lokr(keys) -> bool:
    return any(".lokr_w" in k for k in keys)


def keys_contain_loha(keys) -> bool:
    return any(".hada_w" in k for k in keys)


def keys_are_kohya(keys) -> bool:
    return any(k.startswith(KOHYA_PREFIX) for k in keys)


def detect_lora_prefix(keys) -> str | None:
    keys = list(keys)
    for p in COMMON_LORA_PREFIXES:
        if any(k.startswith(p) for k in keys):
            return p
    return None


def parse_rank_alpha(rank: str | None, alpha: str | None) -> tuple[float, float]:
    """A missing, unparsable or non-positive rank counts as 1 (a zero rank would make alpha / rank non-finite); a
    missing alpha equals the rank (scale 1)."""
    def num(s):
        try:
            return float(s) if s is not None else None
        except ValueError:
            return None
    r = num(rank)
    r = r if r is not None and r > 0 else 1.0
    a = num(alpha)
    return r, (a if a is not None else r)


def split_factor_key(key: str, suffixes) -> tuple[str, str] | None:
    """`a.b.lora_A.weight` with suffix `.lora_A.weight` -> (`a.b`, `lora_A.weight`)."""
    for s in suffixes:
        if key.endswith(s):
            return key[: -len(s)], s[1:]
    return None


def kohya_table(paths) -> dict[str, str]:
    """Underscore-flattened module path -> dotted module path."""
    return {p.replace(".", "_"): p for p in paths}


def resolve_kohya_stem(stem: str, table: dict[str, str]) -> str | None:
    s = stem[len(KOHYA_PREFIX):] if stem.startswith(KOHYA_PREFIX) else stem
    return table.get(s)
