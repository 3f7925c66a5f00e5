"""Validated runtime catalog: the one object a host application composes at start-up (parity:
crates/bundles/runtime-catalog/src/lib.rs:50-135,164-215,299-402,525-600).

A catalog names a platform and a backend and holds the media provider registry, the text-LLM registry, the snapshot
preparer registry and optionally an audio lane (the one sanctioned cross-backend seam). Construction validates:
every descriptor's backend equals the bundle backend; media generators never declare the audio modality; the media
registry passes the weight-free descriptor sweep; LLM descriptors have non-empty identity fields; at least one
snapshot preparer, all on the bundle backend; and, for an audio lane: non-empty backend, every audio generator on the
audio backend with the audio modality, only audio-shaped kinds, no id collision with media generators, its own
descriptor sweep (messages prefixed `audio:`) and at least one preparer on the audio backend."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field

from ..contracts.core_llm.prepare import SnapshotPreparerRegistry
from ..contracts.core_llm.registry import TextLlmRegistry
from ..contracts.errors import InferenceError
from ..contracts.gen_core.generator import Modality
from ..contracts.gen_core.registry import ProviderRegistry

AUDIO_KINDS = ("generator", "voice_embedder", "audio_transform", "transcriber", "audio_embedder")


class RuntimeCatalogError(InferenceError):
    pass


@dataclass
class AudioSection:
    backend: str
    registry: ProviderRegistry
    preparers: SnapshotPreparerRegistry


@dataclass
class RuntimeCatalogSnapshot:
    platform: str
    backend: str
    generator_ids: list[str] = field(default_factory=list)
    transform_ids: list[str] = field(default_factory=list)
    trainer_ids: list[str] = field(default_factory=list)
    captioner_ids: list[str] = field(default_factory=list)
    image_embedder_ids: list[str] = field(default_factory=list)
    text_embedder_ids: list[str] = field(default_factory=list)
    text_llm_ids: list[str] = field(default_factory=list)
    snapshot_preparer_backends: list[str] = field(default_factory=list)
    audio_backend: str | None = None
    audio_generator_ids: list[str] = field(default_factory=list)
    audio_voice_embedder_ids: list[str] = field(default_factory=list)
    audio_transform_ids: list[str] = field(default_factory=list)
    audio_transcriber_ids: list[str] = field(default_factory=list)
    audio_embedder_ids: list[str] = field(default_factory=list)
    audio_snapshot_preparer_backends: list[str] = field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(asdict(self), sort_keys=True)


class RuntimeCatalog:
    def __init__(self, platform: str, backend: str, media: ProviderRegistry, text: TextLlmRegistry,
                 preparers: SnapshotPreparerRegistry, audio: AudioSection | None = None):
        self.platform, self.backend = platform, backend
        self._media, self._text, self._preparers, self._audio = media, text, preparers, audio

    @staticmethod
    def try_new(platform, backend, media, text, preparers) -> "RuntimeCatalog":
        c = RuntimeCatalog(platform, backend, media, text, preparers)
        c._validate()
        return c

    @staticmethod
    def try_new_with_audio(platform, backend, media, text, preparers, audio: AudioSection) -> "RuntimeCatalog":
        c = RuntimeCatalog(platform, backend, media, text, preparers, audio)
        c._validate()
        return c

    def media(self) -> ProviderRegistry:
        return self._media

    def text(self) -> TextLlmRegistry:
        return self._text

    def preparers(self) -> SnapshotPreparerRegistry:
        return self._preparers

    def audio(self) -> AudioSection | None:
        return self._audio

    # ---- validation ---------------------------------------------------------------------------------------
    def _validate(self) -> None:
        errors: list[str] = []
        if not self.platform:
            errors.append("runtime platform is empty")
        if not self.backend:
            errors.append("runtime backend is empty")
        errors.extend(self._media.descriptor_conformance_errors())
        for kind, label in (("generator", "generator"), ("transform", "transform"), ("trainer", "trainer"),
                            ("captioner", "captioner"), ("image_embedder", "image embedder"),
                            ("text_embedder", "text embedder")):
            for reg in self._media.registrations(kind):
                d = reg.descriptor()
                if d.backend != self.backend:
                    errors.append(f"{label} '{d.id}' uses backend '{d.backend}' in the '{self.backend}' runtime")
        for reg in self._media.registrations("generator"):
            d = reg.descriptor()
            if d.modality is Modality.AUDIO:
                errors.append(f"media generator '{d.id}' declares the audio modality - audio generators belong to "
                              "the audio lane, not the media registry")
        for reg in self._text.registrations():
            d = reg.descriptor()
            if not d.id or not d.family or not d.backend:
                errors.append("LLM descriptor contains an empty identity field")
            if d.backend != self.backend:
                errors.append(f"LLM '{d.id}' uses backend '{d.backend}' in the '{self.backend}' runtime")
        if not self._preparers.registrations():
            errors.append("runtime has no snapshot preparer")
        for reg in self._preparers.registrations():
            if reg.backend() != self.backend:
                errors.append(f"snapshot preparer '{reg.backend()}' is in the '{self.backend}' runtime")
        if self._audio is not None:
            self._validate_audio(self._audio, errors)
        if errors:
            raise RuntimeCatalogError("; ".join(errors))

    def _validate_audio(self, a: AudioSection, errors: list[str]) -> None:
        if not a.backend:
            errors.append("runtime audio backend is empty")
        errors.extend(f"audio: {e}" for e in a.registry.descriptor_conformance_errors())
        media_ids = set(self._media.ids("generator"))
        for reg in a.registry.registrations("generator"):
            d = reg.descriptor()
            if d.backend != a.backend:
                errors.append(f"audio generator '{d.id}' uses backend '{d.backend}' in the '{a.backend}' audio lane")
            if d.modality is not Modality.AUDIO:
                errors.append(f"audio generator '{d.id}' does not declare the audio modality")
            if d.id in media_ids:
                errors.append(f"audio generator id '{d.id}' collides with a media generator id")
        for kind in ("voice_embedder", "audio_transform", "transcriber", "audio_embedder"):
            for reg in a.registry.registrations(kind):
                d = reg.descriptor()
                if d.backend != a.backend:
                    errors.append(f"audio {kind.replace('_', ' ')} '{d.id}' uses backend '{d.backend}' in the "
                                  f"'{a.backend}' audio lane")
        for kind in ("transform", "trainer", "captioner", "image_embedder", "text_embedder"):
            if a.registry.registrations(kind):
                errors.append(f"audio lane carries {kind.replace('_', ' ')} registrations; only audio-shaped kinds "
                              "may ride the audio seam")
        if not a.preparers.registrations():
            errors.append("runtime audio lane has no snapshot preparer")
        for reg in a.preparers.registrations():
            if reg.backend() != a.backend:
                errors.append(f"audio snapshot preparer '{reg.backend()}' is in the '{a.backend}' audio lane")

    # ---- snapshot -------------------------------------------------------------------------------------------
    def snapshot(self) -> RuntimeCatalogSnapshot:
        m, a = self._media, self._audio
        s = RuntimeCatalogSnapshot(
            platform=self.platform, backend=self.backend, generator_ids=m.ids("generator"),
            transform_ids=m.ids("transform"), trainer_ids=m.ids("trainer"), captioner_ids=m.ids("captioner"),
            image_embedder_ids=m.ids("image_embedder"), text_embedder_ids=m.ids("text_embedder"),
            text_llm_ids=[r.descriptor().id for r in self._text.registrations()],
            snapshot_preparer_backends=[r.backend() for r in self._preparers.registrations()])
        if a is not None:
            s.audio_backend = a.backend
            s.audio_generator_ids = a.registry.ids("generator")
            s.audio_voice_embedder_ids = a.registry.ids("voice_embedder")
            s.audio_transform_ids = a.registry.ids("audio_transform")
            s.audio_transcriber_ids = a.registry.ids("transcriber")
            s.audio_embedder_ids = a.registry.ids("audio_embedder")
            s.audio_snapshot_preparer_backends = [r.backend() for r in a.preparers.registrations()]
        return s
