"""Audio generators on the sm_100a backend against the fp32 oracle backend."""
import pytest


@pytest.mark.gpu
def test_moss_sfx_on_device_tracks_the_oracle_backend(tmp_path):
    """The text-to-audio generator on the sm_100a backend (bf16 DiT on the tensor-core kernels, fp32 decoder) against the
    fp32 oracle backend: same snapshot, seed and request."""
    import numpy as np

    from inference_b200.audio import moss_sfx
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams

    snap = moss_sfx.write_synthetic_snapshot(tmp_path / "sfx", sample_rate=4800)
    req = dict(prompt="rain on a tin roof", steps=2, seed=3, guidance=2.0, audio=AudioParams(target_duration=1.0))
    out = {}
    for backend, prefix in (("b200", ""), ("cpu", "cpu_")):
        g = provider_registry(backend).load(prefix + "moss_sfx_v2", LoadSpec.from_dir(snap))
        t = g.generate(GenerationRequest(**req)).audio
        out[backend] = np.asarray(t.samples, dtype=np.float32)
    assert out["b200"].shape == out["cpu"].shape == (4800,)
    denom = float(np.abs(out["cpu"]).mean()) + 1e-6
    assert float(np.abs(out["b200"] - out["cpu"]).mean()) / denom < 0.25


@pytest.mark.gpu
def test_acestep_on_device_tracks_the_oracle_backend(tmp_path):
    """Text-to-music and a region edit on the sm_100a backend (bf16 condition encoder and DiT on the tensor-core
    kernels, fp32 autoencoder) against the fp32 oracle backend: same snapshot, seed and request."""
    import numpy as np
    import torch

    from inference_b200.audio import acestep
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams, Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import AudioTrack

    snap = acestep.write_synthetic_snapshot(tmp_path / "ace")
    src = torch.randn(480, 2, generator=torch.Generator().manual_seed(9)) * 0.2
    edit = Conditioning(ConditioningKind.AUDIO_EDIT, audio=AudioTrack(48_000, 2, src.reshape(-1).tolist()), mode="inpaint",
                        region=(0.0025, 0.0075))
    reqs = {"t2m": dict(prompt="calm piano", steps=2, seed=3, audio=AudioParams(target_duration=0.1, lyrics="la la", bpm=90.0)),
            "inpaint": dict(prompt="calm piano", steps=2, seed=3, audio=AudioParams(), conditioning=[edit])}
    for name, req in reqs.items():
        out = {}
        for backend, prefix in (("b200", ""), ("cpu", "cpu_")):
            g = provider_registry(backend).load(prefix + "acestep_v15_turbo", LoadSpec.from_dir(snap))
            out[backend] = np.asarray(g.generate(GenerationRequest(**req)).audio.samples, dtype=np.float32)
        assert out["b200"].shape == out["cpu"].shape, name
        denom = float(np.abs(out["cpu"]).mean()) + 1e-6
        assert float(np.abs(out["b200"] - out["cpu"]).mean()) / denom < 0.25, name
    keep = out["b200"].reshape(-1, 2)[:120]
    assert np.array_equal(keep, src.numpy()[:120])                     # outside the window the source survives bit for bit


@pytest.mark.gpu
def test_moss_tts_realtime_on_device(tmp_path):
    """The streaming text-to-speech generator on the sm_100a backend: the codec (bf16 stages through the tensor-core GEMM)
    tracks the fp32 codec on the same frames in both directions' shapes, and a streamed request yields chunks that
    concatenate to the returned track (sampled tokens are not compared across precisions: one flipped draw changes the
    rest of the utterance)."""
    import torch

    from inference_b200.audio import moss_tts_realtime as M
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams
    from inference_b200.contracts.gen_core.runtime import WeightsSource

    model, codec = M.write_synthetic_snapshot(tmp_path / "m")
    frames = torch.randint(0, 8, (20, 4), generator=torch.Generator().manual_seed(0)).tolist()
    ref = M.MossAudioCodec(codec, 4, "cpu").decode_frames(frames)
    dev = M.MossAudioCodec(codec, 4, "cuda")
    got = dev.decode_frames(frames)
    assert got.shape == ref.shape == (20 * 24,)
    assert float((got - ref).abs().mean()) / (float(ref.abs().mean()) + 1e-6) < 0.1
    assert len(dev.encode(ref, 24_000)) == 20
    spec = LoadSpec.from_dir(model)
    spec.components["codec"] = WeightsSource.dir(codec)
    gen = provider_registry("b200").load("moss_tts_realtime", spec)
    chunks = []
    track = gen.generate_streaming(GenerationRequest(prompt="hello there how are you", seed=3, audio=AudioParams(target_duration=1.6)),
                                   lambda p: None, chunks.append).audio
    assert track.sample_rate == 24_000 and len(track.samples) > 0 and len(track.samples) % 24 == 0
    assert sum((c.samples for c in chunks), []) == track.samples
