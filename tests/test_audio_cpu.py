"""Audio commons (STFT, mel, WAV) and the Whisper model / decoder against Hugging Face on a tiny random config."""
import math

import pytest
import torch

from inference_b200.audio import dsp, mel, wav
from inference_b200.contracts.gen_core.media import AudioTrack


def test_hann_stft_istft_round_trip_and_known_spectrum():
    w = dsp.hann_window(8)
    assert abs(float(w[0])) < 1e-7 and abs(float(w[4]) - 1) < 1e-6
    assert all(abs(float(w[k] - w[8 - k])) < 1e-6 for k in range(1, 8))
    n_fft, hop = 64, 16
    t = torch.arange(2000) / 2000
    x = torch.sin(2 * math.pi * 40 * t) + 0.3 * torch.sin(2 * math.pi * 150 * t)
    sp = dsp.stft(x, n_fft, hop, dsp.hann_window(n_fft))
    assert sp.n_bins == 33 and sp.n_frames == 1 + 2000 // hop and sp.re.shape == (33, sp.n_frames)
    ref = torch.stft(x, n_fft, hop, window=dsp.hann_window(n_fft), center=True, pad_mode="reflect", return_complex=True)
    torch.testing.assert_close(torch.complex(sp.re, sp.im), ref, atol=1e-4, rtol=1e-4)
    y = dsp.istft(sp.magnitude(), sp.phase(), sp.n_frames, n_fft, hop, dsp.hann_window(n_fft))
    assert y.numel() == 2000 and float((y - x).abs().max()) < 1e-3
    for bad in (lambda: dsp.stft(x, 60, hop, dsp.hann_window(60)), lambda: dsp.stft(x, n_fft, 0, dsp.hann_window(n_fft)),
                lambda: dsp.stft(x[:10], n_fft, hop, dsp.hann_window(n_fft)),
                lambda: dsp.stft(x, n_fft, hop, dsp.hann_window(32)),
                lambda: dsp.istft(torch.zeros(5), torch.zeros(5), 2, n_fft, hop, dsp.hann_window(n_fft))):
        with pytest.raises(dsp.AudioError):
            bad()
    up = dsp.nearest_upsample1d(torch.tensor([[[10.0, 20.0, 30.0]]]), 2)
    assert up.flatten().tolist() == [10, 10, 20, 20, 30, 30]
    x3 = torch.randn(2, 3, 5)
    assert torch.equal(dsp.nearest_upsample1d(x3, 3), torch.nn.functional.interpolate(x3, scale_factor=3, mode="nearest"))


def test_mel_filterbanks():
    for hz in (0.0, 100.0, 440.0, 8000.0, 11025.0):
        assert abs(mel.mel_to_hz(mel.hz_to_mel(hz)) - hz) < 0.5
    fb = mel.MelFilterbank.new(24_000, 2048, 80, 0.0, 12_000.0)
    assert (fb.n_mels, fb.n_bins) == (80, 1025) and fb.weights.shape == (80, 1025)
    assert float(fb.weights.min()) >= 0 and float(fb.weights.max()) <= 1 and bool((fb.weights.amax(1) > 0).all())
    peaks = fb.weights.argmax(1)
    assert bool((peaks[1:] >= peaks[:-1]).all())
    out = fb.apply(torch.ones(1025 * 3), 3)
    assert out.shape == (80, 3)
    with pytest.raises(dsp.AudioError):
        fb.apply(torch.ones(7), 3)
    with pytest.raises(dsp.AudioError):
        mel.MelFilterbank.new(16_000, 512, 40, 100.0, 9000.0)
    from transformers.audio_utils import mel_filter_bank
    ref = mel_filter_bank(num_frequency_bins=201, num_mel_filters=80, min_frequency=0.0, max_frequency=8000.0,
                          sampling_rate=16000, norm="slaney", mel_scale="slaney")
    assert float((torch.from_numpy(ref).T.float() - mel.slaney_filterbank(16000, 400, 80)).abs().max()) < 1e-6


def test_wav_pcm16_round_trip():
    import struct

    b = wav.encode_wav_pcm16(AudioTrack(24_000, 1, [0.0, 1.0, -1.0, 0.5]))
    assert len(b) == 52 and b[:4] == b"RIFF" and b[8:16] == b"WAVEfmt " and b[36:40] == b"data"
    assert struct.unpack("<I", b[4:8])[0] == 44 and struct.unpack("<HHIIHH", b[20:36]) == (1, 1, 24000, 48000, 2, 16)
    assert struct.unpack("<4h", b[44:]) == (0, 32767, -32767, 16383)
    assert struct.unpack("<2h", wav.encode_wav_pcm16(AudioTrack(8000, 1, [2.0, -3.0]))[44:]) == (32767, -32767)
    t = wav.decode_wav_pcm16(wav.encode_wav_pcm16(AudioTrack(16_000, 2, [0.25, -0.25, 0.5, -0.5])))
    assert (t.sample_rate, t.channels) == (16_000, 2) and all(abs(a - b) < 1e-4 for a, b in
                                                              zip(t.samples, [0.25, -0.25, 0.5, -0.5]))
    for bad in (AudioTrack(0, 1, [0.0]), AudioTrack(8000, 0, [0.0]), AudioTrack(8000, 2, [0.0, 0.1, 0.2])):
        with pytest.raises(dsp.AudioError):
            wav.encode_wav_pcm16(bad)
    with pytest.raises(dsp.AudioError):
        wav.decode_wav_pcm16(b"nope")


def _tiny_whisper():
    from transformers import WhisperConfig as HfCfg, WhisperForConditionalGeneration

    torch.manual_seed(0)
    hc = HfCfg(vocab_size=200, num_mel_bins=80, d_model=64, encoder_layers=2, encoder_attention_heads=4,
               decoder_layers=2, decoder_attention_heads=4, encoder_ffn_dim=128, decoder_ffn_dim=128,
               max_source_positions=1500, max_target_positions=64, pad_token_id=0, bos_token_id=1, eos_token_id=2,
               decoder_start_token_id=3, suppress_tokens=[5, 6], begin_suppress_tokens=None)
    hf = WhisperForConditionalGeneration(hc).eval()
    return hc, hf


def test_whisper_features_and_model_match_hugging_face():
    from transformers import WhisperFeatureExtractor

    from inference_b200.audio import whisper as W

    g = torch.Generator().manual_seed(0)
    pcm = torch.randn(16_000 * 3, generator=g) * 0.1
    ref = WhisperFeatureExtractor()(pcm.numpy(), sampling_rate=16_000, return_tensors="pt").input_features[0]
    got = W.log_mel_spectrogram(pcm)
    assert got.shape == ref.shape == (80, 3000)
    assert float((got - ref).abs().max()) < 2e-3
    hc, hf = _tiny_whisper()
    cfg = W.WhisperConfig.from_json(hc.to_dict())
    assert cfg.suppress_tokens == [5, 6] and cfg.d_model == 64
    model = W.WhisperModel(cfg, dict(hf.state_dict()), "cpu")
    mel_in = got.unsqueeze(0)
    toks = torch.tensor([[3, 10, 11, 12, 13]])
    with torch.no_grad():
        out = hf(input_features=mel_in, decoder_input_ids=toks)
    audio = model.encode(mel_in)
    torch.testing.assert_close(audio, out.encoder_last_hidden_state, atol=2e-4, rtol=2e-4)
    lg = model.logits(model.decode(toks, audio, True))
    torch.testing.assert_close(lg, out.logits, atol=2e-4, rtol=2e-4)
    # incremental decode through the caches equals the full pass
    model.reset_kv_cache()
    model.decode(toks[:, :2], audio, True)
    model.decode(toks[:, :4], audio, False)
    last = model.logits(model.decode(toks, audio, False))
    torch.testing.assert_close(last[:, -1], out.logits[:, -1], atol=2e-4, rtol=2e-4)
    assert W.resample_to_16k(torch.zeros(2400), 24_000).numel() == 1600
    assert W.to_mono(torch.tensor([1.0, 3.0, 2.0, 4.0]), 2).tolist() == [2.0, 3.0]


class _Tok:
    """Token table: 0..99 text tokens ("w<i>"), then Whisper's control tokens."""
    names = ["<|endoftext|>", "<|startoftranscript|>", "<|en|>", "<|de|>", "<|translate|>", "<|transcribe|>",
             "<|notimestamps|>"]

    def token_to_id(self, t):
        return 100 + self.names.index(t) if t in self.names else None

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(f"w{i}" for i in ids if i < 100)


def test_whisper_decoder_windows_timestamps_and_cancel():
    from inference_b200.audio import whisper as W
    from inference_b200.contracts.errors import Canceled

    hc, hf = _tiny_whisper()
    cfg = W.WhisperConfig.from_json(hc.to_dict())
    model = W.WhisperModel(cfg, dict(hf.state_dict()), "cpu")
    tok = _Tok()
    dec = W.WhisperDecoder(model, tok, timestamps=True)
    assert dec.timestamp_seconds(dec.no_timestamps) is None and abs(dec.timestamp_seconds(dec.no_timestamps + 51) - 1.0) < 1e-6
    assert dec.suppress[5] == float("-inf") and dec.suppress[dec.no_timestamps] == float("-inf") and dec.suppress[7] == 0
    with pytest.raises(W.AudioError):
        dec.language_token("xx")
    assert dec.language_token("de") == 103
    # segment assembly from a scripted token stream (timestamps at 0.0 / 1.0 / 2.5 s, window offset 30 s)
    ts = lambda s: dec.no_timestamps + 1 + int(round(s / 0.02))
    texts, segs = [], []
    dec._append_window([ts(0.0), 1, 2, ts(1.0), ts(1.0), 3, ts(2.5), 4, dec.eot], 30.0, True, texts, segs)
    assert [(round(s.start, 2), round(s.end, 2), s.text) for s in segs] == [(30.0, 31.0, "w1 w2"), (31.0, 32.5, "w3"),
                                                                           (32.5, 32.5, "w4")]
    assert texts == ["w1 w2", "w3", "w4"]
    mel_in = torch.randn(1, 80, 3200, generator=torch.Generator().manual_seed(1)) * 0.1      # two windows
    out = dec.run(mel_in, dec.language_token("en"), False, True, 0.0, 0, 6)
    assert out.tokens <= 12 and out.finish_reason in ("stop_token", "max_tokens")
    again = dec.run(mel_in, dec.language_token("en"), False, True, 0.0, 0, 6)
    assert again.text == out.text and again.tokens == out.tokens
    sampled = dec.run(mel_in[:, :, :3000], None, True, False, 1.0, 7, 4)
    assert sampled.tokens <= 4 and sampled.segments == []
    assert dec.detect_language(mel_in[:, :, :3000]) in (102, 103)
    with pytest.raises(Canceled):
        dec.run(mel_in, None, False, True, 0.0, 0, 6, cancel=lambda: True)
    tr = W.WhisperTranscriber(model, tok, "cpu")
    assert tr.descriptor().id == "whisper"
    segs = tr.transcribe(AudioTrack(8000, 2, [0.01 * math.sin(i / 9) for i in range(16000)]), language="en")
    assert isinstance(segs, list)
    with pytest.raises(W.AudioError):
        tr.transcribe(AudioTrack(16_000, 1, []))


def test_audio_catalog_registers_whisper_and_licenses(tmp_path):
    import json

    from inference_b200.audio import catalog
    from inference_b200.contracts.gen_core.runtime import LoadSpec, WeightsSource
    from inference_b200.io.safetensors_io import save_file

    reg = catalog.provider_registry("cpu")
    assert reg.ids("transcriber") == ["whisper"] and reg.descriptor_conformance_errors() == []
    manifest = json.loads(catalog.weight_licenses_manifest())
    assert [r["provider_id"] for r in manifest["model_weight_licenses"]] == ["acestep_v15_turbo", "chatterbox_ve", "clap_htsat_unfused", "kokoro_82m", "moss_sfx_v2", "moss_tts_realtime", "moss_ttsd_v05", "openvoice_v2", "whisper"]
    assert reg.ids() == ["cpu_kokoro_82m", "cpu_moss_sfx_v2", "cpu_moss_ttsd_v05", "cpu_acestep_v15_turbo", "cpu_moss_tts_realtime"] and catalog.can_prepare(["k/config.json", "k/kokoro-v1_0.pth", "k/voices/af_heart.pt"])
    assert catalog.can_prepare(["a/config.json", "a/tokenizer.json", "a/model.safetensors"])
    assert not catalog.can_prepare(["a/config.json", "a/model.safetensors"])
    hc, hf = _tiny_whisper()
    (tmp_path / "config.json").write_text(json.dumps(hc.to_dict()))
    save_file({k: v.contiguous() for k, v in hf.state_dict().items() if k != "proj_out.weight"}, tmp_path / "model.safetensors")
    vocab = {f"w{i}": i for i in range(100)}
    for i, n in enumerate(_Tok.names):
        vocab[n] = 100 + i
    tok = {"version": "1.0", "model": {"type": "BPE", "vocab": vocab, "merges": []},
           "added_tokens": [{"id": 100 + i, "content": n, "special": True, "single_word": False, "lstrip": False,
                             "rstrip": False, "normalized": False} for i, n in enumerate(_Tok.names)]}
    (tmp_path / "tokenizer.json").write_text(json.dumps(tok))
    tr = reg.load_kind("transcriber", "whisper", LoadSpec.from_dir(tmp_path))
    out = tr.transcribe_full(AudioTrack(16_000, 1, [0.01 * math.sin(i / 7) for i in range(8000)]), language="en",
                             max_new_tokens=4)
    assert out.tokens <= 4
    with pytest.raises(Exception):
        reg.load_kind("transcriber", "whisper", LoadSpec(weights=WeightsSource.file(tmp_path / "model.safetensors")))


def test_chatterbox_voice_encoder(tmp_path):
    from inference_b200.audio import catalog, voice_encoder as ve
    from inference_b200.contracts.gen_core.runtime import LoadSpec, WeightsSource
    from inference_b200.io.safetensors_io import save_file

    torch.manual_seed(0)
    lstm = torch.nn.LSTM(40, 256, num_layers=3, batch_first=True)
    proj = torch.nn.Linear(256, 256)
    w = {f"lstm.{k}": v.detach() for k, v in lstm.state_dict().items()}
    w.update({"proj.weight": proj.weight.detach(), "proj.bias": proj.bias.detach()})
    enc = ve.SpeakerEncoder(w)
    mel = torch.rand(57, 40)
    with torch.no_grad():
        ref = torch.relu(proj(lstm(mel[None])[1][0][-1, 0]))
    torch.testing.assert_close(enc.forward_block(mel), ref, atol=1e-5, rtol=1e-5)
    short = enc.embed_mel_frames(mel)
    assert abs(float(short.norm()) - 1) < 1e-5
    long_mel = torch.rand(400, 40)
    starts = [0, 80, 160, 240]
    want = ve.l2_normalize(sum(enc.forward_block(long_mel[s:s + 160]) for s in starts) / 4)
    torch.testing.assert_close(enc.embed_mel_frames(long_mel), want)
    odd = enc.embed_mel_frames(torch.rand(401, 40))            # a ragged tail adds one partial ending at the last frame
    assert odd.shape == (256,)
    # front end
    quiet = torch.full((1600,), 0.001)
    assert abs(10 * math.log10(float((ve.normalize_volume(quiet) ** 2).mean())) + 30) < 1e-3
    loud = torch.full((1600,), 0.5)
    assert torch.equal(ve.normalize_volume(loud), loud)
    m = ve.wav_to_mel_frames(torch.sin(torch.arange(16000) * 0.05) * 0.1, 16000)
    assert m.shape == (101, 40) and float(m.min()) >= 0
    assert ve.wav_to_mel_frames(torch.zeros(10), 16000).shape[0] == 0
    assert abs(ve.cosine_similarity([1, 0], [-1, 0]) + 1) < 1e-6 and ve.cosine_similarity([0, 0], [1, 1]) == 0.0
    # provider through the audio catalog (a single passed-in file)
    save_file({k: v.contiguous() for k, v in w.items()}, tmp_path / "ve.safetensors")
    reg = catalog.provider_registry("cpu")
    assert reg.ids("voice_embedder") == ["chatterbox_ve"]
    emb = reg.load_kind("voice_embedder", "chatterbox_ve", LoadSpec(weights=WeightsSource.file(tmp_path / "ve.safetensors")))
    track = AudioTrack(24_000, 2, [0.05 * math.sin(i / 11) for i in range(24_000)])
    a, b = emb.embed(track), emb.embed(track)
    assert len(a) == 256 and a == b and abs(sum(x * x for x in a) - 1) < 1e-4
    with pytest.raises(Exception):
        reg.load_kind("voice_embedder", "chatterbox_ve", LoadSpec.from_dir(tmp_path))
    with pytest.raises(dsp.AudioError):
        emb.embed(AudioTrack(16_000, 1, []))


def test_audio_providers_pass_their_conformance_suites():
    from inference_b200.audio import voice_encoder as ve, whisper as W
    from inference_b200.testkit.aux_suites import (ConformanceFailure, TranscriberProfile, transcriber_conformance,
                                                   voice_embedder_conformance)

    hc, hf = _tiny_whisper()
    model = W.WhisperModel(W.WhisperConfig.from_json(hc.to_dict()), dict(hf.state_dict()), "cpu")
    transcriber_conformance(W.WhisperTranscriber(model, _Tok(), "cpu"), TranscriberProfile())
    torch.manual_seed(1)
    lstm, proj = torch.nn.LSTM(40, 256, num_layers=3), torch.nn.Linear(256, 256)
    w = {f"lstm.{k}": v.detach() for k, v in lstm.state_dict().items()}
    w.update({"proj.weight": proj.weight.detach(), "proj.bias": proj.bias.detach()})
    voice_embedder_conformance(ve.ChatterboxVoiceEmbedder(ve.SpeakerEncoder(w), "cpu"))

    class Broken(ve.ChatterboxVoiceEmbedder):          # a provider that returns garbage for empty input
        def embed(self, audio):
            return [0.0] * 256 if not audio.samples else super().embed(audio)
    with pytest.raises(ConformanceFailure, match="degenerate"):
        voice_embedder_conformance(Broken(ve.SpeakerEncoder(w), "cpu"))


def _tiny_clap():
    from transformers import ClapAudioConfig as HA, ClapConfig, ClapModel, ClapTextConfig as HT

    torch.manual_seed(0)
    ac = HA(spec_size=64, num_mel_bins=16, patch_size=4, patch_stride=[4, 4], patch_embeds_hidden_size=16, depths=[2, 2],
            num_attention_heads=[2, 4], window_size=4, hidden_size=32, projection_dim=12, enable_fusion=False)
    tc = HT(vocab_size=120, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
            max_position_embeddings=40, projection_dim=12, pad_token_id=1)
    hc = ClapConfig(text_config=tc.to_dict(), audio_config=ac.to_dict(), projection_dim=12)
    hf = ClapModel(hc).eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "relative_position_bias_table" in n:
                p.copy_(torch.randn_like(p) * 0.5)
        hf.audio_model.audio_encoder.batch_norm.running_mean.copy_(torch.randn(16) * 0.1)
        hf.audio_model.audio_encoder.batch_norm.running_var.copy_(0.5 + torch.rand(16))
    return hc, hf


def test_clap_towers_match_hugging_face():
    from inference_b200.audio import clap as C

    hc, hf = _tiny_clap()
    d = hc.to_dict()
    acfg = C.ClapAudioConfig.from_json(d)
    acfg.patch_stride = 4
    assert acfg.depths == [2, 2] and acfg.projection_dim == 12 and acfg.window_size == 4
    sd = dict(hf.state_dict())
    tower = C.ClapAudioTower(acfg, sd)
    feats = torch.randn(2, 1, 256, 16)                  # 256 frames x 16 mels -> 64 x 64 image (shifted windows in use)
    with torch.no_grad():
        ref = hf.get_audio_features(input_features=feats)
        ref = ref if isinstance(ref, torch.Tensor) else ref.pooler_output
        pooled = hf.audio_model(input_features=feats).pooler_output
    torch.testing.assert_close(tower.pooled(feats), pooled, atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(tower.embed(feats), torch.nn.functional.normalize(ref, dim=-1), atol=2e-4, rtol=2e-4)
    short = torch.randn(1, 1, 100, 16)                  # fewer frames: stretched bicubically to the model's width
    with torch.no_grad():
        ref = hf.audio_model(input_features=short).pooler_output
    torch.testing.assert_close(tower.pooled(short), ref, atol=2e-4, rtol=2e-4)
    text = C.ClapTextTower(C.ClapTextConfig.from_json(d), sd)
    ids = torch.tensor([[0, 5, 6, 7, 2, 1, 1], [0, 9, 2, 1, 1, 1, 1]])
    with torch.no_grad():
        ref = hf.get_text_features(input_ids=ids, attention_mask=(ids != 1).long())
        ref = ref if isinstance(ref, torch.Tensor) else ref.pooler_output
    torch.testing.assert_close(text.embed(ids), torch.nn.functional.normalize(ref, dim=-1), atol=2e-4, rtol=2e-4)


def test_clap_front_end_and_provider():
    from transformers import ClapFeatureExtractor

    from inference_b200.audio import clap as C
    from inference_b200.testkit.aux_suites import vector_embedder_conformance

    g = torch.Generator().manual_seed(3)
    wav = torch.randn(48_000 * 2, generator=g) * 0.05
    fe = ClapFeatureExtractor(truncation="rand_trunc", padding="repeatpad", frequency_min=50, frequency_max=14_000)
    ref = torch.from_numpy(fe(wav.numpy(), sampling_rate=48_000, return_tensors="np")["input_features"])[0, 0]
    got = C.log_mel_db(C.fit_length(wav))
    assert got.shape == ref.shape == (1001, 64)
    assert float((got - ref).abs().max()) < 2e-2        # dB scale; fp32 vs float64 STFT
    assert C.fit_length(torch.arange(5.0), 12).tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4, 0, 0]
    assert C.fit_length(torch.arange(20.0), 12).numel() == 12
    assert C.resample_linear(torch.zeros(2400), 24_000).numel() == 4800

    hc, hf = _tiny_clap()

    class Tiny(C.ClapAudioTower):                       # the tiny tower takes 16 mel bins: fold the 64-band front end
        def embed(self, feats):
            return super().embed(feats[:, :, :256, :].reshape(feats.shape[0], 1, 256, 16, 4).mean(-1))
    acfg = C.ClapAudioConfig.from_json(hc.to_dict())
    acfg.patch_stride = 4
    sd = dict(hf.state_dict())

    class Tok:
        def encode(self, t, add_special_tokens=True):
            return [0] + [int(x) for x in t.split()] + [2]
    from inference_b200.audio import catalog

    assert catalog.provider_registry("cpu").ids("audio_embedder") == ["clap_htsat_unfused"]
    emb = C.ClapAudioEmbedder(Tiny(acfg, sd), C.ClapTextTower(C.ClapTextConfig.from_json(hc.to_dict()), sd), Tok(), "cpu")
    clips = [AudioTrack(24_000, 2, [0.05 * math.sin(i / 13) for i in range(12_000)]),
             AudioTrack(48_000, 1, [0.02 * math.sin(i / 5) for i in range(30_000)])]
    vector_embedder_conformance(emb, clips)
    tv = emb.embed_text(["5 6 7", "9"])
    assert len(tv) == 2 and len(tv[0]) == 12 and abs(sum(x * x for x in tv[0]) - 1) < 1e-4
    assert emb.descriptor().id == "clap_htsat_unfused" and emb.descriptor().extra["joint_text"]
    with pytest.raises(C.AudioError):
        emb.embed([AudioTrack(48_000, 1, [])])
