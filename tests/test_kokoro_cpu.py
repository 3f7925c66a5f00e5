"""Kokoro: building blocks against torch.nn modules / closed forms, the harmonic source and the tiny STFT pair,
phonemisation, the frame-count law of the whole pipeline, and the audio-generator conformance suite."""
import math

import torch
import torch.nn.functional as F

from inference_b200.audio import kokoro as K


def test_blocks_match_torch_modules():
    torch.manual_seed(0)
    lstm = torch.nn.LSTM(6, 5, batch_first=True, bidirectional=True)
    w = _W = K._W({"l." + k: v.detach() for k, v in lstm.state_dict().items()}, "cpu")
    x = torch.randn(1, 9, 6)
    assert torch.allclose(w.bilstm(x, "l"), lstm(x)[0], atol=1e-5)
    # old-style weight norm folds to g * v / ||v||
    v, g = torch.randn(4, 3, 5), torch.rand(4, 1, 1) + 0.5
    wn = K._W({"c.weight_v": v, "c.weight_g": g, "c.bias": torch.zeros(4)}, "cpu")
    ref = torch.nn.utils.weight_norm(torch.nn.Conv1d(3, 4, 5), name="weight")
    ref.weight_v.data, ref.weight_g.data, ref.bias.data = v, g, torch.zeros(4)
    xin = torch.randn(1, 3, 20)
    assert torch.allclose(wn.conv(xin, "c"), ref(xin), atol=1e-5)
    # AdaIN: instance norm then (1 + gamma) x + beta from the style
    fc_w, fc_b, s, h = torch.randn(8, 3), torch.randn(8), torch.randn(1, 3), torch.randn(1, 4, 11)
    a = K._W({"n.fc.weight": fc_w, "n.fc.bias": fc_b}, "cpu").adain(h, s, "n")
    gb = s @ fc_w.t() + fc_b
    want = F.instance_norm(h, eps=1e-5) * (1 + gb[:, :4, None]) + gb[:, 4:, None]
    assert torch.allclose(a, want, atol=1e-5)
    x4 = torch.tensor([-1.0, 0.0, 1.0, 2.0])
    assert torch.allclose(K.gelu_new(x4), torch.tensor([-0.15880801, 0.0, 0.841192, 1.9545977]), atol=1e-6)


def test_harmonic_source_and_stft_pair():
    gen = torch.Generator().manual_seed(1)
    f0 = torch.tensor([0.0, 0.0, 220.0, 220.0, 220.0])
    lw = torch.zeros(1, 9)
    lw[0, 0] = 1.0
    src = K.harmonic_source(f0, 300, lw, 0.0, gen)
    assert src.shape == (1500,)
    unv, voi = src[:500], src[800:1500]
    assert unv.abs().max() < 0.25 and voi.abs().max() > 0.07           # unvoiced: noise only (sigma 0.033); voiced: the 0.1 sine
    # voiced region oscillates at ~220 Hz: count zero crossings over 700 samples at 24 kHz -> ~2 * 220 * 700 / 24000 = 12.8
    zc = int(((voi[:-1] * voi[1:]) < 0).sum())
    assert 9 <= zc <= 20
    x = torch.randn(600)
    mag, ph = K.stft_small(x, 20, 5)
    assert mag.shape == (11, 121)
    assert torch.allclose(K.istft_small(mag, ph, 20, 5), x, atol=1e-4)


def test_phonemisation():
    vocab = {c: i + 1 for i, c in enumerate(" ,.!?abdefhijklmnpstuvwzæɛɪɑʌɹθʃʧŋʤɡAOWYəð")}
    g = K.KokoroG2p({"hello": "həlO", "the": "ðə"}, vocab)
    assert g.phonemize("Hello, the ship!") == "həlO, ðə ʃɪp!"
    assert g.phonemize("həlO wɜld") == "həlO wɜld"                        # an IPA script passes through
    cfg = K.KokoroConfig(vocab=vocab)
    assert cfg.phonemes_to_ids("a ɜ b") == [vocab["a"], vocab[" "], vocab[" "], vocab["b"]]      # unknown symbols drop out


def test_pipeline_frame_law_and_conformance(tmp_path):
    import pytest

    from inference_b200.audio.catalog import provider_registry as audio_registry
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams
    from inference_b200.testkit.audio_generator import AudioProfile, audio_conformance

    snap = K.write_synthetic_snapshot(tmp_path / "kokoro")
    reg = audio_registry("cpu")
    assert "cpu_kokoro_82m" in reg.ids()
    gen = reg.load("cpu_kokoro_82m", LoadSpec.from_dir(snap))
    audio_conformance(gen, AudioProfile(prompt="hello world, the fox!", voice="af_heart", target_duration=0.5))
    pipe = gen.pipeline()
    toks = pipe.cfg.phonemes_to_ids("həlO")
    ref_s = gen.voice_pack("af_heart")[len(toks) - 1][None]
    raw = pipe.raw_durations(toks, ref_s)
    assert raw.shape == (len(toks) + 2,) and (raw > 0).all() and (raw < pipe.cfg.max_dur).all()
    slow = pipe.synthesize(toks, ref_s, 0.5, 3)
    fast = pipe.synthesize(toks, ref_s, 2.0, 3)
    frames = lambda sp: int(torch.round(raw / sp).clamp(min=1).sum())      # noqa: E731
    assert slow.numel() == frames(0.5) * 600 and fast.numel() == frames(2.0) * 600 and slow.numel() > fast.numel()
    out = gen.generate(GenerationRequest(prompt="the fox", seed=1, audio=AudioParams(voice="bf_emma")))
    assert out.audio.sample_rate == 24_000 and out.audio.channels == 1
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(prompt="the fox", seed=1, audio=AudioParams(voice="am_adam")))      # pack not in the snapshot
    with pytest.raises(InferenceError):
        pipe.synthesize(list(range(1, 70)), ref_s, 1.0, 0)                                                # beyond the 64-token context
