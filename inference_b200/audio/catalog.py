"""The audio lane's provider catalog (candle-audio-catalog/src/lib.rs:67-110): an explicit registration list, the
weight-license manifest of the checkpoints those providers load, and the lane's snapshot-preparation predicate."""
from __future__ import annotations

from ..contracts.gen_core.license import WeightLicense, WeightLicenseEntry, weight_licenses_manifest_json
from ..contracts.gen_core.registry import ProviderRegistry, ProviderRegistryBuilder, Registration
from ..contracts.gen_core.runtime import LoadSpec
from ..contracts.gen_core.traits import SimpleDescriptor

WHISPER_LICENSE = WeightLicense("MIT", "MIT License", "https://huggingface.co/openai/whisper-base", "OpenAI", True)


def _whisper_registration(backend: str) -> Registration:
    def load(spec: LoadSpec):
        from .whisper import WhisperTranscriber

        if spec.weights is None or spec.weights.is_file:
            from ..contracts.errors import LoadError

            raise LoadError("whisper: the load spec needs a snapshot directory")
        return WhisperTranscriber.load_dir(spec.weights.path, "cuda" if backend == "b200" else "cpu", backend)

    return Registration(lambda: SimpleDescriptor("whisper", "whisper", backend, {"sample_rate": 16_000}), load)


CHATTERBOX_LICENSE = WeightLicense("MIT", "MIT License", "https://huggingface.co/ResembleAI/chatterbox", "Resemble AI", True)


def _chatterbox_ve_registration(backend: str) -> Registration:
    def load(spec: LoadSpec):
        from ..contracts.errors import LoadError
        from ..io.safetensors_io import load_file
        from .voice_encoder import ChatterboxVoiceEmbedder, SpeakerEncoder

        if spec.weights is None or not spec.weights.is_file:
            raise LoadError("chatterbox_ve: the load spec needs the ve.safetensors file")
        return ChatterboxVoiceEmbedder(SpeakerEncoder(load_file(spec.weights.path), "cuda" if backend == "b200" else "cpu"),
                                       backend)

    return Registration(lambda: SimpleDescriptor("chatterbox_ve", "chatterbox", backend, {"dim": 256}), load)


def register_providers(b: ProviderRegistryBuilder, backend: str) -> ProviderRegistryBuilder:
    b.register("transcriber", _whisper_registration(backend))
    b.register("voice_embedder", _chatterbox_ve_registration(backend))
    return b


def provider_registry(backend: str = "b200") -> ProviderRegistry:
    return register_providers(ProviderRegistryBuilder(), backend).build()


def weight_licenses() -> list[WeightLicenseEntry]:
    return [WeightLicenseEntry("whisper", WHISPER_LICENSE), WeightLicenseEntry("chatterbox_ve", CHATTERBOX_LICENSE)]


def weight_licenses_manifest() -> str:
    return weight_licenses_manifest_json(weight_licenses())


def can_prepare(files: list[str]) -> bool:
    """A Whisper snapshot ships config.json, tokenizer.json and safetensors weights."""
    names = {f.rsplit("/", 1)[-1] for f in files}
    return "config.json" in names and "tokenizer.json" in names and any(n.endswith(".safetensors") for n in names)
