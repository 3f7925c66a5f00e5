"""Tensor-free media contracts: generator trait and request model, load types, registries, the unified sampler
framework, guidance, tiling and memory policy (parity target: crates/contracts/gen-core)."""
from ..errors import Canceled, InferenceError, InvalidRequest, LoadError, Unsupported  # noqa: F401
from .generator import (AudioParams, Capabilities, Conditioning, ConditioningKind, ConversationSession,  # noqa: F401
                        ConversationTurn, GenerationOutput, GenerationPhase, GenerationRequest, Generator, Modality,
                        ModelDescriptor)
from .guidance import GUIDANCE_METHODS, GuidanceMethod, MomentumBuffer, apg, apg_delta, cfg, cfg_rescale  # noqa: F401
from .media import AudioChunk, AudioTrack, Image  # noqa: F401
from .registry import (ModelRegistration, PerComponentBytes, ProviderRegistry, ProviderRegistryBuilder,  # noqa: F401
                       Registration, model_descriptor_errors)
from .runtime import (AdapterKind, AdapterSpec, CancelFlag, LoadPhase, LoadSpec, OffloadPolicy, Precision,  # noqa: F401
                      Progress, ProgressDecoding, ProgressLoading, ProgressStep, Quant, WeightsSource)
from .tiling import (VAE_TILING_PRESETS, MemoryPlan, TilePlan, TilingConfig, budgeted_plan,  # noqa: F401
                     plan_memory_adaptation, plan_tiles, trapezoidal_mask)
from .traits import (AudioEmbedder, AudioTransform, Captioner, ControlBranch, FaceEmbedder, ImageEmbedder,  # noqa: F401
                     SimpleDescriptor, TextEmbedder, Trainer, TrainingConfig, TrainingProgress, Transcriber,
                     Transform, VoiceEmbedder, reject_unknown_components, require_component)
