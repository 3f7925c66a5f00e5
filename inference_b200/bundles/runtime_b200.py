"""The sm_100a runtime bundle (the role of crates/bundles/runtime-cuda/src/lib.rs:3-92): one call composes the
media provider registry, the text-LLM registry and the snapshot preparers of the B200 backend into a validated
catalog. Nothing is discovered at import time; the lists below are the shipped surface."""
from __future__ import annotations

from ..contracts.core_llm.prepare import SnapshotPreparerRegistry, SnapshotPreparerRegistryBuilder
from ..contracts.core_llm.registry import TextLlmRegistry, TextLlmRegistryBuilder
from ..contracts.gen_core.registry import ProviderRegistry
from .catalog import AudioSection, RuntimeCatalog

PLATFORM = "cuda"
BACKEND = "b200"


def provider_registry() -> ProviderRegistry:
    from ..media.catalog import provider_registry as media_registry

    return media_registry(BACKEND)


def text_registry() -> TextLlmRegistry:
    from ..engine.provider import B200_LLAMA, B200_LLAVA, B200_QWEN3_VL

    return TextLlmRegistryBuilder().register(B200_LLAMA).register(B200_LLAVA).register(B200_QWEN3_VL).build()


def snapshot_preparer_registry() -> SnapshotPreparerRegistry:
    from ..io.prepare import registration

    return SnapshotPreparerRegistryBuilder().register(registration(BACKEND)).build()


def audio_section() -> AudioSection:
    """The audio lane: its own provider registry (transcribers, embedders, generators) on the same backend; its
    snapshots are prepared by the lane's preparer list."""
    from ..audio.catalog import provider_registry as audio_registry

    return AudioSection(BACKEND, audio_registry(BACKEND), snapshot_preparer_registry())


def catalog() -> RuntimeCatalog:
    return RuntimeCatalog.try_new_with_audio(PLATFORM, BACKEND, provider_registry(), text_registry(),
                                             snapshot_preparer_registry(), audio_section())
