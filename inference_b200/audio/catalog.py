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


CLAP_LICENSE = WeightLicense("Apache-2.0", "Apache License 2.0", "https://huggingface.co/laion/clap-htsat-unfused",
                             "LAION", True)


def _clap_registration(backend: str) -> Registration:
    def load(spec: LoadSpec):
        import json
        from pathlib import Path

        import torch

        from ..contracts.core_llm.tokenizer import Tokenizer
        from ..contracts.errors import LoadError
        from ..io.safetensors_io import load_dir
        from .clap import ClapAudioConfig, ClapAudioEmbedder, ClapAudioTower, ClapTextConfig, ClapTextTower

        if spec.weights is None or spec.weights.is_file:
            raise LoadError("clap_htsat_unfused: the load spec needs a snapshot directory")
        d = Path(spec.weights.path)
        cfg = json.loads((d / "config.json").read_text())
        w = load_dir(d)
        dev, dtype = ("cuda", torch.bfloat16) if backend == "b200" else ("cpu", torch.float32)
        acfg = ClapAudioConfig.from_json(cfg)
        if isinstance(acfg.patch_stride, (list, tuple)):
            acfg.patch_stride = int(acfg.patch_stride[0])
        text = tok = None
        if (d / "tokenizer.json").is_file() and any(k.startswith("text_model.") for k in w):
            text, tok = ClapTextTower(ClapTextConfig.from_json(cfg), w, dev, dtype), Tokenizer.from_file(d / "tokenizer.json")
        return ClapAudioEmbedder(ClapAudioTower(acfg, w, dev, dtype), text, tok, backend)

    return Registration(lambda: SimpleDescriptor("clap_htsat_unfused", "clap", backend, {"dim": 512, "sample_rate": 48_000}),
                        load)


OPENVOICE_LICENSE = WeightLicense("MIT", "MIT License", "https://huggingface.co/myshell-ai/OpenVoiceV2", "MyShell", True)


def _openvoice_registration(backend: str) -> Registration:
    def load(spec: LoadSpec):
        from ..contracts.errors import LoadError
        from .openvoice import OpenVoiceConverter, OpenVoiceTransform, load_checkpoint

        if spec.weights is None:
            raise LoadError("openvoice_v2: the load spec needs the converter checkpoint (a file or its directory)")
        return OpenVoiceTransform(OpenVoiceConverter(load_checkpoint(spec.weights.path), "cuda" if backend == "b200" else "cpu"),
                                  backend)

    return Registration(lambda: SimpleDescriptor("openvoice_v2", "openvoice", backend, {"sample_rate": 22_050}), load)


def register_providers(b: ProviderRegistryBuilder, backend: str) -> ProviderRegistryBuilder:
    from . import acestep, kokoro, moss_sfx, moss_tts_realtime, moss_ttsd

    b.register_generators([kokoro.registration(backend), moss_sfx.registration(backend), moss_ttsd.registration(backend),
                           acestep.registration(backend), moss_tts_realtime.registration(backend)])
    b.register("transcriber", _whisper_registration(backend))
    b.register("voice_embedder", _chatterbox_ve_registration(backend))
    b.register("audio_embedder", _clap_registration(backend))
    b.register("audio_transform", _openvoice_registration(backend))
    return b


def provider_registry(backend: str = "b200") -> ProviderRegistry:
    return register_providers(ProviderRegistryBuilder(), backend).build()


def weight_licenses() -> list[WeightLicenseEntry]:
    from .kokoro import KOKORO_LICENSE
    from .acestep import ACESTEP_LICENSE
    from .moss_sfx import MOSS_SFX_LICENSE
    from .moss_tts_realtime import MOSS_TTS_REALTIME_LICENSE
    from .moss_ttsd import MOSS_TTSD_LICENSE

    return [WeightLicenseEntry("kokoro_82m", KOKORO_LICENSE), WeightLicenseEntry("moss_sfx_v2", MOSS_SFX_LICENSE), WeightLicenseEntry("moss_ttsd_v05", MOSS_TTSD_LICENSE), WeightLicenseEntry("acestep_v15_turbo", ACESTEP_LICENSE), WeightLicenseEntry("moss_tts_realtime", MOSS_TTS_REALTIME_LICENSE), WeightLicenseEntry("whisper", WHISPER_LICENSE), WeightLicenseEntry("chatterbox_ve", CHATTERBOX_LICENSE),
            WeightLicenseEntry("clap_htsat_unfused", CLAP_LICENSE), WeightLicenseEntry("openvoice_v2", OPENVOICE_LICENSE)]


def weight_licenses_manifest() -> str:
    return weight_licenses_manifest_json(weight_licenses())


def can_prepare(files: list[str]) -> bool:
    """A Whisper snapshot ships config.json, tokenizer.json and safetensors weights."""
    names = {f.rsplit("/", 1)[-1] for f in files}
    if "config.json" in names and ("kokoro-v1_0.pth" in names or "kokoro.safetensors" in names):
        return True                      # Kokoro snapshots carry no tokenizer.json: validated passthrough
    return "config.json" in names and "tokenizer.json" in names and any(n.endswith(".safetensors") for n in names)
