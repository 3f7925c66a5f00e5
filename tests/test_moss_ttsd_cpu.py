"""MOSS-TTSD: configuration checks, the seeded sampler, the delay pattern (shift / un-shift / teacher forcing / drain), the
codec's signal pieces (inverse DFT basis, overlap-add, sinusoids, weight-norm folding) and the generator end to end."""
import math

import pytest
import torch

from inference_b200.audio import moss_ttsd as T


def _cfg(**kw):
    base = dict(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                num_key_value_heads=1, head_dim=16, channels=4, speech_vocab_size=17, speech_pad_token=16,
                speech_token_range=[200, 216], speech_eos_token=218, bos_token_id=219)
    base.update(kw)
    return base


def test_config_rules():
    c = T.MossTtsdConfig.from_json(_cfg())
    assert c.text_pad_id == 219 and c.channels == 4 and c.speech_token_range == (200, 216)
    d = T.MossTtsdConfig.from_json({k: v for k, v in _cfg().items() if k not in ("channels", "speech_vocab_size", "speech_pad_token",
                                                                                 "speech_token_range", "speech_eos_token", "bos_token_id")})
    assert (d.channels, d.speech_vocab_size, d.speech_pad_token, d.speech_eos_token, d.text_pad_id) == (8, 1025, 1024, 152_694, 151_643)
    for bad in (dict(channels=1), dict(speech_vocab_size=0), dict(speech_token_range=[216, 200]), dict(speech_token_range=[200, 204])):
        with pytest.raises(T.LoadError):
            T.MossTtsdConfig.from_json(_cfg(**bad))


def test_seeded_sampler():
    a, b, c = T.Rng(42), T.Rng(42), T.Rng(43)
    sa = [a.next_f32() for _ in range(8)]
    assert sa == [b.next_f32() for _ in range(8)] and sa != [c.next_f32() for _ in range(8)] and all(0.0 <= x < 1.0 for x in sa)
    # SplitMix64 reference value: seed 0 ^ gamma, first output
    r = T.Rng(0)
    z = (0x9E3779B97F4A7C15 * 2) & T.M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & T.M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & T.M64
    assert r.next_u64() == z ^ (z >> 31)
    lg = torch.tensor([0.1, 5.0, 0.2, -1.0])
    assert T.sample(lg.clone(), T.Rng(1), temperature=0.0) == 1
    for _ in range(20):
        assert T.sample(torch.tensor([1.0, 2.0, 9.0, 3.0, 0.5]), T.Rng(7), temperature=1.0, top_k=1, top_p=1.0) == 2
    # top-p drops the unlikely tail: with p = 0.5 only the dominant token survives
    rng = T.Rng(3)
    assert all(T.sample(torch.tensor([4.0, 0.0, 0.0, 0.0]), rng, 1.0, 4, 0.5) == 0 for _ in range(30))
    # frequencies follow the softmax
    rng, counts = T.Rng(5), [0, 0]
    for _ in range(4000):
        counts[T.sample(torch.tensor([0.0, math.log(3.0)]), rng, 1.0, 2, 1.0)] += 1
    assert 0.70 < counts[1] / 4000 < 0.80
    assert T.sample(torch.tensor([float("-inf")] * 3), T.Rng(1), 1.0, 3, 1.0) in (0, 1, 2)


def test_delay_pattern():
    cfg = T.MossTtsdConfig.from_json(_cfg())
    grid = [[(k + 1) % 300] + [16] * 3 for k in range(3)]
    sh = T.shift_grid(grid, cfg)
    assert len(sh) == 3 + 3
    for j in range(4):
        for r, src in enumerate(grid):
            assert sh[j + r][j] == src[j]
    assert sh[3][0] == cfg.text_pad_id
    emitted = [[200 + t, t % 16, (t + 1) % 16, (t + 2) % 16] for t in range(8)]
    clean = T.unshift(emitted, cfg)
    assert len(clean) == 5 and clean[0] == [0, 1, 3, 5] and clean[2] == [2, 3, 5, 7]
    emitted[3][1] = 16                                                 # a pad on a delayed channel drops that frame
    assert len(T.unshift(emitted, cfg)) == 4
    assert T.unshift(emitted[:3], cfg) == []
    assert T.format_dialogue_text("[S1]hi[S2]yo") == "<speaker1>hi<speaker2>yo"
    assert T.script_to_dialogue([{"text": " a ", "speaker": "x"}, {"text": "b", "speaker": "y"}, {"text": "c", "speaker": "x"}]) == "[S1]a[S2]b[S1]c"
    assert T.script_to_dialogue([{"text": "a"}, {"text": "b"}, {"text": "c"}]) == "[S1]a[S2]b[S1]c"


def test_codec_signal_pieces():
    w = T.hann_window(8)
    assert w[0] == 0.0 and w[4] == pytest.approx(1.0) and w[1] == pytest.approx(w[7])
    s = T.sinusoids(5, 8)
    assert s.shape == (5, 8) and s[0, :4].abs().max() == 0.0 and (s[0, 4:] == 1.0).all()
    n = 16
    cos, sin = T.idft_basis(n)
    x = torch.cos(2 * math.pi * 3 * torch.arange(n) / n) + 0.25
    spec = torch.fft.rfft(x)
    assert torch.allclose(spec.real @ cos.t() - spec.imag @ sin.t(), x, atol=1e-5)
    frames = torch.randn(6, 960)
    out = T.overlap_add(frames, T.hann_window(960), 240)
    assert out.numel() == 6 * 240
    # a stream of identical constant frames reconstructs the constant where the windows overlap fully
    const = T.overlap_add(torch.ones(9, 960) * 0.5, T.hann_window(960), 240)
    ws = T.hann_window(960)
    mid = const[960:1200]
    num = sum(ws[k * 240:(k + 1) * 240] for k in range(4))
    den = sum(ws[k * 240:(k + 1) * 240] ** 2 for k in range(4))
    assert torch.allclose(mid, 0.5 * num / den, atol=1e-5)
    v, g = torch.randn(5, 3, 2), torch.rand(5, 1, 1) + 0.5
    folded = T.resolve_weight_norm({"a.weight_v": v, "a.weight_g": g, "a.bias": torch.zeros(5)})
    assert set(folded) == {"a.weight", "a.bias"} and torch.allclose(folded["a.weight"].flatten(1).norm(dim=1), g.flatten(), atol=1e-5)
    with pytest.raises(T.LoadError):
        T.resolve_weight_norm({"a.weight_g": g})


def test_generator_end_to_end(tmp_path):
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams
    from inference_b200.contracts.gen_core.runtime import WeightsSource

    snap, codec = T.write_synthetic_snapshot(tmp_path / "ttsd")
    reg = provider_registry("cpu")
    assert "cpu_moss_ttsd_v05" in reg.ids()
    with pytest.raises(InferenceError, match="codec"):
        reg.load("cpu_moss_ttsd_v05", LoadSpec.from_dir(snap))
    spec = LoadSpec(weights=WeightsSource.dir(snap), components={"codec": WeightsSource.file(codec)})
    gen = reg.load("cpu_moss_ttsd_v05", spec)
    d = gen.descriptor()
    assert d.family == "moss_ttsd" and d.capabilities.supports_multi_speaker and d.capabilities.max_speakers == 2
    assert d.required_components == ["codec"] and d.capabilities.audio_sample_rates == [24_000]
    req = GenerationRequest(prompt="[S1]hello there[S2]fine thanks", seed=7, audio=AudioParams(target_duration=1.0))
    backbone = gen.pipeline()[0]
    cfg = backbone.cfg
    # random weights never stay in the speech range: steer channel 0 into it for a dozen positions per decode, then out
    plain, calls = backbone.channel_logits, {"n": 0}

    def steered(hidden):
        lg = plain(hidden)
        calls["n"] += 1
        if calls["n"] <= 12:
            lg[0][cfg.speech_token_range[0]:cfg.speech_token_range[1]] += 30.0
        else:
            lg[0][5] += 60.0
        return lg

    backbone.channel_logits = steered
    rvq = gen.rvq_frames

    def fresh(r, *a):
        calls["n"] = 0
        return rvq(r, *a)

    gen.rvq_frames = fresh
    frames, stop = gen.rvq_frames(req)
    assert stop == "eos"
    assert stop in ("eos", "budget") and frames
    width0 = cfg.speech_token_range[1] - cfg.speech_token_range[0]
    assert all(len(f) == cfg.channels and f[0] < width0 and all(c < cfg.speech_vocab_size - 1 for c in f[1:]) for f in frames)
    assert gen.rvq_frames(req)[0] == frames                           # the seeded decode is reproducible
    assert gen.rvq_frames(GenerationRequest(**{**req.__dict__, "seed": 8}))[0] != frames
    out = gen.generate(req).audio
    assert out.sample_rate == 24_000 and out.channels == 1 and len(out.samples) == len(frames) * T.SAMPLES_PER_FRAME
    assert all(math.isfinite(x) for x in out.samples[:2000])
    script = GenerationRequest(prompt="", seed=7, audio=AudioParams(script=[{"text": "hello there", "speaker": "a"}, {"text": "fine thanks", "speaker": "b"}]))
    assert gen.rvq_frames(script)[0] == frames                        # the script renders to the same dialogue text
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt="  "))
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt="x", audio=AudioParams(target_duration=301.0)))
    # cancellation between positions is typed
    from inference_b200.contracts.errors import Canceled
    from inference_b200.contracts.gen_core.runtime import CancelFlag

    flag, seen = CancelFlag(), []

    def prog(p):
        seen.append(p)
        if len(seen) >= 2:
            flag.cancel()

    with pytest.raises(Canceled):
        gen.generate(GenerationRequest(**{**req.__dict__, "cancel": flag}), prog)
    assert len(seen) <= 3
    assert T.position_budget(GenerationRequest(prompt="x"), 8) == 125 + 8 and T.position_budget(req, 8) == 64 + 8
