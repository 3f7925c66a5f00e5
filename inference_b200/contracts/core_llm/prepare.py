"""Snapshot preparation contract: format detection, specs, reports and the preparer registry
(core-llm/src/prepare.rs:29-269). "Prepare" converts a checkpoint once (GGUF or safetensors, optionally
quantising) into a self-contained snapshot directory that then loads fast."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable

from ..errors import InferenceError, Unsupported
from .request import Quantize


class ModelFormat(enum.Enum):
    GGUF = "gguf"
    SAFETENSORS = "safetensors"

    def as_str(self) -> str:
        return self.value


def _has_gguf_magic(path: Path) -> bool:
    try:
        with open(path, "rb") as f:
            return f.read(4) == b"GGUF"
    except OSError:
        return False


def detect_format(source: str | Path) -> ModelFormat:
    p = Path(source)
    if p.is_file():
        if _has_gguf_magic(p):
            return ModelFormat.GGUF
        if p.suffix == ".gguf":
            return ModelFormat.GGUF
        if p.suffix == ".safetensors":
            return ModelFormat.SAFETENSORS
        raise Unsupported(f"cannot prepare '{p}': not a GGUF (no `GGUF` magic) nor a `*.safetensors` file")
    if p.is_dir():
        if (p / "config.json").is_file():
            return ModelFormat.SAFETENSORS
        if any(c.suffix == ".gguf" for c in p.iterdir()):
            return ModelFormat.GGUF
        raise Unsupported(f"cannot prepare '{p}': directory has no config.json (HF snapshot) and no *.gguf")
    raise Unsupported(f"cannot prepare '{p}': path does not exist or is neither a file nor a directory")


@dataclass(frozen=True)
class PrepareSpec:
    source: Path
    out_dir: Path
    quantize: Quantize | None = None

    @staticmethod
    def dense(source, out_dir) -> "PrepareSpec":
        return PrepareSpec(Path(source), Path(out_dir), None)

    @staticmethod
    def quantized(source, out_dir, quantize: Quantize) -> "PrepareSpec":
        return PrepareSpec(Path(source), Path(out_dir), quantize)


@dataclass(frozen=True)
class PrepareReport:
    input_format: ModelFormat
    quantized: Quantize | None
    out_dir: Path
    num_tensors: int
    passthrough: bool


@dataclass(frozen=True)
class SnapshotPreparerRegistration:
    backend: Callable[[], str]
    can_prepare: Callable[[PrepareSpec], bool]
    prepare: Callable[[PrepareSpec], PrepareReport]


class SnapshotPreparerRegistryBuilder:
    def __init__(self):
        self._regs: list[SnapshotPreparerRegistration] = []

    def register(self, reg: SnapshotPreparerRegistration) -> "SnapshotPreparerRegistryBuilder":
        self._regs.append(reg)
        return self

    def extend(self, regs: Iterable[SnapshotPreparerRegistration]) -> "SnapshotPreparerRegistryBuilder":
        self._regs.extend(regs)
        return self

    def build(self) -> "SnapshotPreparerRegistry":
        seen = set()
        for r in self._regs:
            b = r.backend()
            if b in seen:
                raise InferenceError(f"duplicate snapshot preparer backend '{b}' in explicit registry")
            seen.add(b)
        return SnapshotPreparerRegistry(tuple(self._regs))


class SnapshotPreparerRegistry:
    def __init__(self, regs: tuple[SnapshotPreparerRegistration, ...]):
        self._regs = regs

    def registrations(self) -> tuple[SnapshotPreparerRegistration, ...]:
        return self._regs

    def prepare_snapshot(self, spec: PrepareSpec) -> PrepareReport:
        for r in self._regs:
            if r.can_prepare(spec):
                return r.prepare(spec)
        try:
            fmt = f"format={detect_format(spec.source).as_str()}"
        except InferenceError:
            fmt = "unrecognized source format"
        names = ", ".join(sorted({r.backend() for r in self._regs})) or "(none)"
        raise Unsupported(f"no linked backend can prepare a snapshot from '{spec.source}' ({fmt}); "
                          f"linked preparers: {names}")
