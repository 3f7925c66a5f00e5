"""Explicit, immutable media provider registry (gen-core/src/registry.rs:51-646): ten registration kinds, a
builder that rejects duplicate ids per kind and can refuse a quantisation tier registry-wide, weightless
descriptor conformance, and per-component weight footprints read from safetensors headers."""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterable

from ..errors import InferenceError, Unsupported
from .generator import ConditioningKind, Generator, Modality, ModelDescriptor
from .runtime import LoadSpec, Quant

KINDS = ("generator", "transform", "audio_transform", "trainer", "captioner", "transcriber", "image_embedder",
         "text_embedder", "voice_embedder", "audio_embedder")


@dataclass(frozen=True)
class Registration:
    """descriptor() is weightless; load(spec) builds the provider. `footprint(spec)` is optional."""
    descriptor: Callable[[], Any]
    load: Callable[[LoadSpec], Any]
    footprint: Callable[[LoadSpec], "PerComponentBytes | None"] | None = None


ModelRegistration = Registration


@dataclass
class PerComponentBytes:
    components: dict[str, int] = field(default_factory=dict)

    def total(self) -> int:
        return sum(self.components.values())

    @staticmethod
    def from_root_subdirs(root: Path, subdirs: dict[str, str]) -> "PerComponentBytes":
        from ...io.safetensors_io import header_bytes_and_count

        out = {}
        for name, sub in subdirs.items():
            d = Path(root) / sub
            if d.exists():
                try:
                    out[name] = header_bytes_and_count(d)[0]
                except InferenceError:
                    out[name] = 0
        return PerComponentBytes(out)


def _check_names(errs: list[str], ctx: str, what: str, names: Iterable[str]) -> None:
    seen = set()
    for n in names:
        if not n or n != n.strip() or any(ch.isspace() for ch in n):
            errs.append(f"{ctx}: {what} name {n!r} is blank or contains whitespace")
        if n in seen:
            errs.append(f"{ctx}: duplicate {what} {n!r}")
        seen.add(n)


def model_descriptor_errors(d: ModelDescriptor) -> list[str]:
    """Weights-free descriptor sanity: identity fields, non-zero bounds, clean name lists, no duplicate
    conditioning kinds, no video conditioning on an image-only model."""
    errs: list[str] = []
    ctx = f"generator '{d.id}'"
    for k, v in (("id", d.id), ("family", d.family), ("backend", d.backend)):
        if not v or v != v.strip():
            errs.append(f"{ctx}: {k} is empty or padded")
    caps = d.capabilities
    if caps.max_count == 0:
        errs.append(f"{ctx}: max_count is 0 - every request would be rejected")
    if d.modality is not Modality.AUDIO:
        if caps.min_size == 0 or caps.max_size == 0:
            errs.append(f"{ctx}: min_size={caps.min_size} max_size={caps.max_size} - size bounds left at the default 0")
        elif caps.min_size > caps.max_size:
            errs.append(f"{ctx}: min_size {caps.min_size} > max_size {caps.max_size}")
    _check_names(errs, ctx, "sampler", caps.samplers)
    _check_names(errs, ctx, "scheduler", caps.schedulers)
    _check_names(errs, ctx, "guidance_method", caps.supported_guidance_methods)
    seen = set()
    for k in caps.conditioning:
        if k in seen:
            errs.append(f"{ctx}: duplicate conditioning kind {k.name}")
        seen.add(k)
        if k in (ConditioningKind.KEYFRAME, ConditioningKind.VIDEO_SYNC) and d.modality is Modality.IMAGE:
            errs.append(f"{ctx}: advertises video conditioning {k.name} but modality is Image")
    _check_names(errs, ctx, "required_component", d.required_components)
    return errs


class ProviderRegistryBuilder:
    def __init__(self):
        self._regs: dict[str, list[Registration]] = {k: [] for k in KINDS}
        self._rejected: list[tuple[Quant, str]] = []

    def register(self, kind: str, reg: Registration) -> "ProviderRegistryBuilder":
        if kind not in self._regs:
            raise InferenceError(f"unknown registration kind {kind!r}")
        self._regs[kind].append(reg)
        return self

    def register_generators(self, regs: Iterable[Registration]) -> "ProviderRegistryBuilder":
        self._regs["generator"].extend(regs)
        return self

    def reject_quant(self, quant: Quant, reason: str) -> "ProviderRegistryBuilder":
        self._rejected.append((quant, reason))
        return self

    def build(self) -> "ProviderRegistry":
        for kind, regs in self._regs.items():
            seen = set()
            for r in regs:
                i = r.descriptor().id
                if i in seen:
                    raise InferenceError(f"duplicate {kind.replace('_', ' ')} id '{i}' in explicit registry")
                seen.add(i)
        return ProviderRegistry({k: tuple(v) for k, v in self._regs.items()}, tuple(self._rejected))


class ProviderRegistry:
    def __init__(self, regs: dict[str, tuple[Registration, ...]], rejected: tuple[tuple[Quant, str], ...]):
        self._regs, self._rejected = regs, rejected

    def registrations(self, kind: str = "generator") -> tuple[Registration, ...]:
        return self._regs[kind]

    def ids(self, kind: str = "generator") -> list[str]:
        return [r.descriptor().id for r in self._regs[kind]]

    def find(self, kind: str, provider_id: str) -> Registration | None:
        for r in self._regs[kind]:
            if r.descriptor().id == provider_id:
                return r
        return None

    def _load(self, kind: str, provider_id: str, spec: LoadSpec):
        r = self.find(kind, provider_id)
        if r is None:
            raise InferenceError(f"no {kind.replace('_', ' ')} registered for id '{provider_id}'")
        if spec.quantize is not None:
            for q, reason in self._rejected:
                if q is spec.quantize:
                    raise Unsupported(f"{provider_id}: quantisation {q.value} is rejected by this registry: {reason}")
        return r.load(spec)

    def load(self, provider_id: str, spec: LoadSpec) -> Generator:
        return self._load("generator", provider_id, spec)

    def load_kind(self, kind: str, provider_id: str, spec: LoadSpec):
        return self._load(kind, provider_id, spec)

    def footprint(self, provider_id: str, spec: LoadSpec) -> PerComponentBytes | None:
        r = self.find("generator", provider_id)
        if r is None:
            raise InferenceError(f"no generator registered for id '{provider_id}'")
        return r.footprint(spec) if r.footprint else None

    def descriptor_conformance_errors(self) -> list[str]:
        errs: list[str] = []
        for r in self._regs["generator"]:
            errs += model_descriptor_errors(r.descriptor())
        for kind in KINDS[1:]:
            for r in self._regs[kind]:
                d = r.descriptor()
                for k in ("id", "family", "backend"):
                    v = getattr(d, k, "")
                    if not v or v != v.strip():
                        errs.append(f"{kind} '{getattr(d, 'id', '?')}': {k} is empty or padded")
        return errs
