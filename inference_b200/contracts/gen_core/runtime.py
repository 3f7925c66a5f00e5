"""Load-time types shared by every media provider (gen-core/src/runtime.rs:18-453): weight sources (local paths
only, never a hub fetch), quantisation / precision / offload policy, adapter specs, cancel flag and progress."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from pathlib import Path

from ..core_llm.cancel import CancelFlag  # noqa: F401  (one CancelFlag type across both contracts)


class Quant(enum.Enum):
    Q4 = "q4"
    Q8 = "q8"
    NVFP4 = "nvfp4"


class Precision(enum.Enum):
    BF16 = "bf16"
    F16 = "f16"
    F32 = "f32"


class OffloadPolicy(enum.Enum):
    RESIDENT = "resident"      # every component stays on the device (default on 180 GB parts)
    SEQUENTIAL = "sequential"  # text encoder -> (free) -> DiT + VAE, one resident at a time


@dataclass(frozen=True)
class WeightsSource:
    path: Path
    is_file: bool = False

    @staticmethod
    def dir(path) -> "WeightsSource":
        return WeightsSource(Path(path), False)

    @staticmethod
    def file(path) -> "WeightsSource":
        return WeightsSource(Path(path), True)


class AdapterKind(enum.Enum):
    LORA = "lora"
    LOKR = "lokr"


@dataclass
class AdapterSpec:
    path: Path
    scale: float = 1.0
    kind: AdapterKind = AdapterKind.LORA
    pass_scales: list[float] | None = None
    moe_expert: str | None = None


@dataclass
class LoadSpec:
    weights: WeightsSource | None = None
    quantize: Quant | None = None
    precision: Precision | None = None
    control: WeightsSource | None = None
    extra_controls: list[WeightsSource] = field(default_factory=list)
    ip_adapter: WeightsSource | None = None
    adapters: list[AdapterSpec] = field(default_factory=list)
    pid: WeightsSource | None = None
    identity: WeightsSource | None = None
    text_encoder: WeightsSource | None = None
    offload_policy: OffloadPolicy = OffloadPolicy.RESIDENT
    components: dict[str, WeightsSource] = field(default_factory=dict)

    @staticmethod
    def from_dir(path) -> "LoadSpec":
        return LoadSpec(weights=WeightsSource.dir(path))


class LoadPhase(enum.Enum):
    TEXT_ENCODER = "text_encoder"
    TRANSFORMER = "transformer"
    VAE = "vae"
    ADAPTERS = "adapters"


@dataclass(frozen=True)
class ProgressStep:
    current: int   # 1-based
    total: int


@dataclass(frozen=True)
class ProgressDecoding:
    pass


@dataclass(frozen=True)
class ProgressLoading:
    phase: LoadPhase


Progress = ProgressStep | ProgressDecoding | ProgressLoading
