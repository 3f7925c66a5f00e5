"""The other provider traits of the media contract, each with its descriptor (parity: gen-core/src/train.rs,
caption.rs, transform.rs, transcribe.rs, image_embed.rs, text_embed.rs, voice_embed.rs, audio_embed.rs,
audio_transform.rs, face.rs, control.rs). They are tensor-free interfaces; engines implement them."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

from ..errors import InferenceError, Unsupported
from .media import AudioTrack, Image
from .runtime import CancelFlag, WeightsSource


@dataclass
class SimpleDescriptor:
    id: str
    family: str
    backend: str
    extra: dict[str, Any] = field(default_factory=dict)


@dataclass
class TrainingConfig:
    dataset_dir: Path | None = None
    output_dir: Path | None = None
    steps: int = 1000
    batch_size: int = 1
    grad_accum: int = 1
    learning_rate: float = 1e-4
    lr_schedule: str = "constant"
    warmup_steps: int = 0
    rank: int = 16
    alpha: float = 16.0
    adapter: str = "lora"
    seed: int = 0
    gradient_checkpointing: bool = False
    save_every: int = 0
    resume: Path | None = None
    cancel: CancelFlag = field(default_factory=CancelFlag)


@dataclass
class TrainingProgress:
    step: int
    total: int
    loss: float
    learning_rate: float = 0.0
    checkpoint: Path | None = None


class Trainer(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def validate(self, cfg: TrainingConfig) -> None: ...
    @abc.abstractmethod
    def train(self, cfg: TrainingConfig, on_progress: Callable[[TrainingProgress], None]) -> Path: ...


class Captioner(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def caption(self, image: Image, prompt: str | None = None, max_new_tokens: int = 256) -> str: ...


class Transform(abc.ABC):
    """Image -> image utility (upscaler, depth, segmentation...)."""
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def apply(self, image: Image, params: dict[str, Any] | None = None) -> Image: ...


class AudioTransform(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def apply(self, audio: AudioTrack, params: dict[str, Any] | None = None) -> AudioTrack: ...


@dataclass
class TranscriptSegment:
    start: float
    end: float
    text: str


class Transcriber(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def transcribe(self, audio: AudioTrack, language: str | None = None) -> list[TranscriptSegment]: ...


class ImageEmbedder(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def embed(self, images: list[Image]) -> list[list[float]]: ...


class TextEmbedder(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def embed(self, texts: list[str]) -> list[list[float]]: ...


class VoiceEmbedder(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def embed(self, audio: AudioTrack) -> list[float]: ...


class AudioEmbedder(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> SimpleDescriptor: ...
    @abc.abstractmethod
    def embed(self, audio: list[AudioTrack]) -> list[list[float]]: ...


@dataclass
class FaceDetection:
    bbox: tuple[float, float, float, float]
    landmarks: list[tuple[float, float]]
    score: float
    embedding: list[float] | None = None


class FaceEmbedder(abc.ABC):
    """Face detection + identity embedding (gen-core/src/face.rs:40-61). Results are ordered largest face first."""
    @abc.abstractmethod
    def detect(self, image: Image) -> list[FaceDetection]:
        """Boxes and landmarks only (embeddings stay None): the cheap path."""

    def analyze(self, image: Image) -> list[FaceDetection]:
        """Every face with its raw embedding."""
        raise NotImplementedError

    def largest_face(self, image: Image) -> FaceDetection:
        faces = self.analyze(image)
        if not faces:
            raise InferenceError("no face detected")
        return faces[0]


class ControlBranch(abc.ABC):
    """An auxiliary conditioning network (ControlNet-style) a generator may host."""
    @abc.abstractmethod
    def kind(self) -> str: ...
    @abc.abstractmethod
    def residuals(self, latents: Any, control_image: Image, timestep: float, scale: float) -> Any: ...


def require_component(components: dict[str, WeightsSource], name: str, model_id: str) -> WeightsSource:
    if name not in components:
        raise InferenceError(f"{model_id}: required component '{name}' was not provided in LoadSpec.components")
    return components[name]


def reject_unknown_components(components: dict[str, WeightsSource], known: list[str], model_id: str) -> None:
    for k in components:
        if k not in known:
            raise Unsupported(f"{model_id}: unknown component '{k}' (known: {known})")
