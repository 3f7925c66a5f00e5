"""The media generator contract (gen-core/src/generator.rs:17-1416): request, conditioning, outputs, descriptors,
capabilities and the shared validation floor every provider starts from."""
from __future__ import annotations

import abc
import enum
import math
from dataclasses import dataclass, field, fields
from typing import Any, Callable

from ..errors import InferenceError, Unsupported
from .media import AudioTrack, Image
from .runtime import CancelFlag, Progress, Quant

MAX_STEPS = 100_000
MAX_FRAMES = 1_000_000
MAX_FPS = 100_000
MAX_DURATION_SECS = 1_000_000.0


class Modality(enum.Enum):
    IMAGE = "image"
    VIDEO = "video"
    BOTH = "both"
    AUDIO = "audio"


class ConditioningKind(enum.Enum):
    REFERENCE = "reference"
    MULTI_REFERENCE = "multi_reference"
    MASK = "mask"
    CONTROL = "control"
    DEPTH = "depth"
    POSE = "pose"
    IP_ADAPTER = "ip_adapter"
    IDENTITY = "identity"
    KEYFRAME = "keyframe"
    FIRST_FRAME = "first_frame"
    LAST_FRAME = "last_frame"
    AUDIO_EDIT = "audio_edit"
    VIDEO_SYNC = "video_sync"
    VOICE_REFERENCE = "voice_reference"
    REFERENCE_AUDIO = "reference_audio"
    VOICE_EMBEDDING = "voice_embedding"
    REDUX_REFS = "redux_refs"
    VIDEO_CLIP = "video_clip"                 # frames of a source clip (video -> video, upscaling)
    CONTROL_CLIP = "control_clip"             # frames of a control signal (pose / depth video)
    CONVERSATION_HISTORY = "conversation_history"


@dataclass
class Conditioning:
    """One conditioning input: its kind plus the payload that kind carries (image, mask, frames, region ...)."""
    kind: ConditioningKind
    image: Image | None = None
    images: list[Image] = field(default_factory=list)
    frames: list[Image] = field(default_factory=list)
    mask_frames: list[Image] = field(default_factory=list)        # CONTROL_CLIP: one mask per frame (white = generate)
    audio: AudioTrack | None = None
    strength: float | None = None
    frame_index: int | None = None
    mode: str | None = None
    region: tuple[float, float | None] | None = None   # (start_secs, end_secs)
    turns: list = field(default_factory=list)           # CONVERSATION_HISTORY: list[ConversationTurn]


@dataclass
class ConversationTurn:
    """One turn of a multi-turn conversation: role "user" or "assistant", its text, and its audio when the turn is
    provided context (a user turn always carries audio; an assistant turn without audio is synthesised)."""
    role: str = "assistant"
    text: str = ""
    audio: AudioTrack | None = None


class ConversationSession(abc.ABC):
    """Stateful counterpart of a CONVERSATION_HISTORY request: the model's cross-turn state stays live, each `step`
    advances by one turn and returns that turn's audio. For the same conversation and seed a session emits the samples
    a single request carrying all turns emits (gen-core/src/generator.rs:120-168)."""

    @abc.abstractmethod
    def step(self, turn: ConversationTurn, on_chunk=lambda c: None, on_progress=lambda p: None) -> AudioTrack: ...

    def finish(self) -> None:
        return None


@dataclass
class AudioParams:
    voice: str | None = None
    language: str | None = None
    target_duration: float | None = None
    sample_rate: int | None = None
    bpm: float | None = None
    musical_key: str | None = None
    lyrics: str | None = None
    script: list[dict] | None = None    # [{text, speaker, style}]


@dataclass
class GenerationPhase:
    steps: int
    guidance: float | None = None
    adapters: list[tuple[int, float | None]] = field(default_factory=list)


@dataclass
class GenerationRequest:
    prompt: str = ""
    negative_prompt: str | None = None
    width: int = 1024
    height: int = 1024
    count: int = 1
    seed: int | None = None
    steps: int | None = None
    guidance: float | None = None
    true_cfg: float | None = None
    timestep_to_start_cfg: int | None = None
    sampler: str | None = None
    scheduler: str | None = None
    scheduler_shift: float | None = None
    guidance_method: str | None = None
    guidance_eta: float | None = None
    guidance_momentum: float | None = None
    guidance_norm_threshold: float | None = None
    conditioning: list[Conditioning] = field(default_factory=list)
    strength: float | None = None
    control_scale: float | None = None
    text_style_gain: float | None = None
    image_guidance: float | None = None
    frames: int | None = None
    fps: int | None = None
    duration: float | None = None
    video_mode: str | None = None
    trim_first_frames: int | None = None
    motion_bucket_id: float | None = None
    noise_aug_strength: float | None = None
    decode_chunk_size: int | None = None
    conditioning_fps: int | None = None
    softness: float | None = None
    enhance_prompt: bool = False
    use_uncensored_enhancer: bool = False
    enhance_max_tokens: int | None = None
    enhance_temperature: float | None = None
    use_pid: bool = False
    pid_capture_sigma: float | None = None
    audio: AudioParams | None = None
    phases: list[GenerationPhase] | None = None
    cancel: CancelFlag = field(default_factory=CancelFlag)

    def ensure_finite_floats(self) -> None:
        """Every float knob (present and future) must be finite: a NaN passes range checks silently."""
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, float) and not math.isfinite(v):
                raise InferenceError(f"{f.name} must be finite (got {v})")
        if self.audio is not None:
            for name in ("target_duration", "bpm"):
                v = getattr(self.audio, name)
                if isinstance(v, float) and not math.isfinite(v):
                    raise InferenceError(f"audio.{name} must be finite (got {v})")
        for c in self.conditioning:
            if c.strength is not None and not math.isfinite(c.strength):
                raise InferenceError("conditioning strength must be finite")
            if c.region is not None and any(x is not None and not math.isfinite(x) for x in c.region):
                raise InferenceError("conditioning region must be finite")


@dataclass
class GenerationOutput:
    images: list[Image] = field(default_factory=list)
    video_frames: list[Image] = field(default_factory=list)
    fps: int | None = None
    audio: AudioTrack | None = None

    @property
    def kind(self) -> str:
        if self.video_frames:
            return "video"
        if self.images:
            return "images"
        return "audio" if self.audio is not None else "empty"


@dataclass
class Capabilities:
    supports_negative_prompt: bool = False
    supports_guidance: bool = False
    supports_true_cfg: bool = False
    conditioning: list[ConditioningKind] = field(default_factory=list)
    supports_lora: bool = False
    supports_lokr: bool = False
    samplers: list[str] = field(default_factory=list)
    schedulers: list[str] = field(default_factory=list)
    supported_guidance_methods: list[str] = field(default_factory=list)
    min_size: int = 0
    max_size: int = 0
    max_count: int = 0
    mac_only: bool = False
    audio_sample_rates: list[int] = field(default_factory=list)
    max_audio_duration_secs: float | None = None
    audio_voices: list[str] = field(default_factory=list)
    audio_languages: list[str] = field(default_factory=list)
    audio_edit_modes: list[str] = field(default_factory=list)
    supports_streaming: bool = False
    supports_multi_speaker: bool = False
    max_speakers: int | None = None
    supports_conversation_history: bool = False
    supports_conversation_session: bool = False
    supported_quants: tuple[Quant, ...] = ()
    supports_kv_cache: bool = False
    requires_sigma_shift: bool = False
    supports_sequential_offload: bool = False

    def accepts(self, kind: ConditioningKind) -> bool:
        return kind in self.conditioning

    def validate_request(self, mid: str, req: GenerationRequest) -> None:
        self._validate(mid, req, True)

    def validate_request_skip_size(self, mid: str, req: GenerationRequest) -> None:
        self._validate(mid, req, False)

    def validate_request_audio(self, mid: str, req: GenerationRequest) -> None:
        self._validate(mid, req, False)

    def _validate(self, mid: str, req: GenerationRequest, check_size: bool) -> None:
        def msg(text: str):
            raise InferenceError(f"{mid}: {text}")

        def gap(text: str):
            raise Unsupported(f"{mid}: {text}")

        assert self.max_count > 0 and (not check_size or self.max_size > 0), \
            f"{mid}: Capabilities max_count/max_size left at 0 - the descriptor forgot its bounds"
        if req.count == 0 or req.count > self.max_count:
            msg(f"count {req.count} out of range 1..={self.max_count}")
        if req.steps == 0:
            msg("steps must be >= 1 (an explicit 0 renders undenoised noise)")
        if req.steps is not None and req.steps > MAX_STEPS:
            msg(f"steps {req.steps} exceeds the sanity cap {MAX_STEPS}")
        if req.frames is not None and req.frames > MAX_FRAMES:
            msg(f"frames {req.frames} exceeds the sanity cap {MAX_FRAMES}")
        if req.fps is not None and req.fps > MAX_FPS:
            msg(f"fps {req.fps} exceeds the sanity cap {MAX_FPS}")
        if req.duration is not None and req.duration > MAX_DURATION_SECS:
            msg(f"duration {req.duration}s exceeds the sanity cap {MAX_DURATION_SECS}s")
        a = req.audio
        if a is not None:
            d = a.target_duration
            if d is not None:
                if d <= 0.0:
                    msg(f"audio.target_duration must be > 0 (got {d}s)")
                if d > MAX_DURATION_SECS:
                    msg(f"audio.target_duration {d}s exceeds the sanity cap {MAX_DURATION_SECS}s")
                if self.max_audio_duration_secs is not None and d > self.max_audio_duration_secs:
                    msg(f"audio.target_duration {d}s exceeds the supported maximum {self.max_audio_duration_secs}s")
            if a.bpm is not None and a.bpm <= 0.0:
                msg(f"audio.bpm must be > 0 (got {a.bpm})")
            if a.sample_rate is not None and a.sample_rate not in self.audio_sample_rates:
                gap(f"unsupported audio.sample_rate {a.sample_rate} (supported: {self.audio_sample_rates})")
            if a.voice is not None and a.voice not in self.audio_voices:
                gap(f"unsupported audio.voice {a.voice!r} (supported: {self.audio_voices})")
            if a.language is not None and a.language not in self.audio_languages:
                gap(f"unsupported audio.language {a.language!r} (supported: {self.audio_languages})")
            if a.script is not None:
                if not self.supports_multi_speaker:
                    gap("a multi-speaker audio.script is not supported")
                if not a.script:
                    msg("audio.script must not be empty")
                speakers = {s.get("speaker") for s in a.script if s.get("speaker")}
                if self.max_speakers is not None and len(speakers) > self.max_speakers:
                    msg(f"audio.script names {len(speakers)} speakers, more than the supported {self.max_speakers}")
                if self.audio_voices:
                    for sp in speakers:
                        if sp not in self.audio_voices:
                            gap(f"unsupported audio.script speaker {sp!r} (supported: {self.audio_voices})")
        if check_size and (req.width < self.min_size or req.height < self.min_size or req.width > self.max_size
                           or req.height > self.max_size):
            msg(f"size {req.width}x{req.height} outside supported range {self.min_size}..={self.max_size}")
        if req.negative_prompt is not None and not self.supports_negative_prompt:
            gap("negative prompts are not supported")
        if req.guidance is not None and not self.supports_guidance:
            gap("guidance is not supported")
        if req.true_cfg is not None and not self.supports_true_cfg:
            gap("true_cfg is not supported")
        req.ensure_finite_floats()
        if req.sampler is not None and req.sampler not in self.samplers:
            gap(f"unsupported sampler {req.sampler!r} (supported: {self.samplers})")
        if req.scheduler is not None and req.scheduler not in self.schedulers:
            gap(f"unsupported scheduler {req.scheduler!r} (supported: {self.schedulers})")
        if req.guidance_method is not None and req.guidance_method not in self.supported_guidance_methods:
            gap(f"unsupported guidance_method {req.guidance_method!r} (supported: {self.supported_guidance_methods})")
        for c in req.conditioning:
            if not self.accepts(c.kind):
                gap(f"{c.kind.name} conditioning is not supported")
        for c in req.conditioning:
            if c.kind is ConditioningKind.AUDIO_EDIT:
                if c.mode not in self.audio_edit_modes:
                    gap(f"unsupported audio edit mode {c.mode!r} (supported: {self.audio_edit_modes})")
                if c.region is not None:
                    start, end = c.region
                    if start < 0.0:
                        msg(f"audio edit region start {start}s must be >= 0")
                    if end is not None and end <= start:
                        msg(f"audio edit region end {end}s must be > start {start}s")
            if c.kind is ConditioningKind.CONVERSATION_HISTORY:
                if not self.supports_conversation_history:
                    gap("conversation histories are not supported")
                if not c.turns:
                    msg("a conversation history must carry at least one turn")
                for i, t in enumerate(c.turns):
                    if t.role not in ("user", "assistant"):
                        msg(f"conversation turn {i}: unknown role {t.role!r}")
                    if not t.text.strip():
                        msg(f"conversation turn {i}: empty text")
                    if t.role == "user" and t.audio is None:
                        msg(f"conversation turn {i}: a user turn must carry its audio")
            if c.kind is ConditioningKind.VIDEO_SYNC and not c.frames:
                msg("VideoSync conditioning carries no frames - a video->audio clip must have at least one frame")


@dataclass
class ModelDescriptor:
    id: str
    family: str
    backend: str
    modality: Modality
    capabilities: Capabilities
    required_components: list[str] = field(default_factory=list)


class Generator(abc.ABC):
    @abc.abstractmethod
    def descriptor(self) -> ModelDescriptor: ...

    @abc.abstractmethod
    def validate(self, req: GenerationRequest) -> None: ...

    @abc.abstractmethod
    def generate(self, req: GenerationRequest, on_progress: Callable[[Progress], None]) -> GenerationOutput:
        """Emits exactly `steps` ProgressStep events (1-based) per image, then ProgressDecoding; a cancelled request
        raises Canceled."""

    def generate_streaming(self, req: GenerationRequest, on_progress, on_chunk) -> GenerationOutput:
        out = self.generate(req, on_progress)
        if out.audio is not None:
            on_chunk(out.audio)
        return out

    def open_conversation(self, req: GenerationRequest | None = None) -> ConversationSession:
        """`req` carries what stays constant across the conversation (seed, audio knobs, a reference voice, the cancel
        flag); the turns arrive through the session's `step`."""
        raise Unsupported(f"{self.descriptor().id}: conversation sessions are not supported")
