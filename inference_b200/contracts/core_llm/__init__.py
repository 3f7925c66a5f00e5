"""Tensor-free text-LLM contracts: provider trait, request / output model, capabilities, typed errors,
registries, snapshot preparation and the stream-text policies (parity target: crates/contracts/core-llm)."""
from ..errors import (BackendError, Canceled, ConfigError, InferenceError, InvalidRequest, IoError, LoadError,  # noqa: F401
                      Unsupported)
from .cancel import CancelFlag  # noqa: F401
from .capabilities import TextLlmCapabilities, TextLlmDescriptor  # noqa: F401
from .constraint import Constraint, ConstraintDecodeTable, JsonConstraint, JsonState  # noqa: F401
from .detok import IncrementalDetok  # noqa: F401
from .message import Content, ImageRef, Message, Role, Text, VideoRef  # noqa: F401
from .output import Channel, DoneEvent, FinishReason, StreamEvent, TextLlmOutput, TokenEvent, Usage  # noqa: F401
from .prepare import (ModelFormat, PrepareReport, PrepareSpec, SnapshotPreparerRegistration,  # noqa: F401
                      SnapshotPreparerRegistry, SnapshotPreparerRegistryBuilder, detect_format)
from .registry import ModelRequirements, TextLlmRegistration, TextLlmRegistry, TextLlmRegistryBuilder  # noqa: F401
from .request import LoadSpec, Quantize, Sampling, TextLlmRequest, ThinkingMode  # noqa: F401
from .stop import StopChunk, StopMatcher  # noqa: F401
from .text_llm import TextLlm  # noqa: F401
from .thinking import ThinkingSegmenter, ThinkingSpan  # noqa: F401
from .tool import ToolCall, ToolCallSegmenter, ToolSpec  # noqa: F401
from .template import ChatMlTemplate, ChatTemplate, JinjaChatTemplate, Llama3Template, RenderOptions  # noqa: F401
from .tokenizer import Tokenizer  # noqa: F401
