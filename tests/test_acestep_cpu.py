"""ACE-Step: prompt assembly, the shifted schedule, the DiT against a convolution-based restatement, the Oobleck
autoencoder against torch.nn layers with weight norm, the scalar quantiser, stitching rules, edit windows and the
audio-generator conformance suite with region edits and a cover."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.audio import acestep as A


def test_prompt_weaves_metadata_in_a_fixed_order():
    meta = A.Metadata(128.0, "C minor", "4", "en")
    assert A.build_prompt("  upbeat   electronic\ndance track ", meta) == \
        "upbeat electronic dance track, bpm: 128, key: C minor, time signature: 4, language: en"
    assert A.build_prompt("ambient pad", A.Metadata()) == "ambient pad"
    assert A.build_prompt("lofi", A.Metadata(bpm=90.0)) == "lofi, bpm: 90"
    assert A.build_prompt("lofi", A.Metadata(bpm=90.5, key="  ")) == "lofi, bpm: 90.5"


def test_schedule():
    assert A.flow_sigmas(4, 1.0) == pytest.approx([1.0, 0.75, 0.5, 0.25, 0.0], abs=1e-12)
    s = A.flow_sigmas(8, 3.0)
    assert s[0] == 1.0 and s[-1] == 0.0 and s[4] > A.flow_sigmas(8, 1.0)[4] and len(s) == 9
    assert abs(A.flow_sigmas(2, 3.0)[1] - 0.75) < 1e-12
    assert len(A.flow_sigmas(0, 3.0)) == 2


def _restated_dit(cfg, w, hidden, context_latents, t, enc):
    lin = lambda x, p: F.linear(x, w[p + ".weight"], w.get(p + ".bias"))       # noqa: E731
    rms = lambda v, g: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g   # noqa: E731
    H, KV, D, d, p = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size, cfg.patch_size
    T = hidden.shape[1]
    x = torch.cat([context_latents, hidden], -1)
    if T % p:
        x = torch.cat([x, torch.zeros(1, p - T % p, x.shape[2])], 1)
    x = F.conv1d(x.transpose(1, 2), w["proj_in_conv.weight"], w["proj_in_conv.bias"], stride=p).transpose(1, 2)
    N = x.shape[1]

    def temb(prefix, tt):
        half = A.FREQ_DIM // 2
        ang = tt * 1000.0 * torch.exp(-torch.arange(half, dtype=torch.float64) * math.log(10000.0) / half)
        s = torch.cat([ang.cos(), ang.sin()]).float()[None]
        e = lin(F.silu(lin(s, prefix + "linear_1")), prefix + "linear_2")
        return e, lin(F.silu(e), prefix + "time_proj")

    (e1, p1), (e2, p2) = temb("time_embed.", t), temb("time_embed_r.", 0.0)
    e, tproj = e1 + e2, (p1 + p2).view(1, 6, d)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    th = (torch.arange(N, dtype=torch.float64)[:, None] * inv).float()

    def rope(v):                                   # [1, h, N, D], halves
        a, b = v[..., : D // 2], v[..., D // 2:]
        return torch.cat([a * th.cos() - b * th.sin(), b * th.cos() + a * th.sin()], -1)

    def attn(pfx, xq, src, rot, mask):
        q = rms(lin(xq, pfx + "to_q").view(1, -1, H, D), w[pfx + "norm_q.weight"]).transpose(1, 2)
        k = rms(lin(src, pfx + "to_k").view(1, -1, KV, D), w[pfx + "norm_k.weight"]).transpose(1, 2)
        v = lin(src, pfx + "to_v").view(1, -1, KV, D).transpose(1, 2)
        if rot:
            q, k = rope(q), rope(k)
        k, v = k.repeat_interleave(H // KV, 1), v.repeat_interleave(H // KV, 1)
        s = q @ k.transpose(-1, -2) / math.sqrt(D)
        if mask is not None:
            s = s + mask
        return lin((torch.softmax(s, -1) @ v).transpose(1, 2).reshape(1, -1, H * D), pfx + "to_out.0")

    i = torch.arange(N)
    sliding = torch.where((i[:, None] - i[None, :]).abs() <= cfg.sliding_window, 0.0, float("-inf"))
    ctx = lin(enc, "condition_embedder")
    for li in range(cfg.num_hidden_layers):
        b = f"layers.{li}."
        m = w[b + "scale_shift_table"] + tproj
        h = rms(x, w[b + "self_attn_norm.weight"]) * (1 + m[:, 1:2]) + m[:, 0:1]
        x = x + attn(b + "self_attn.", h, h, True, sliding if cfg.layer_types[li] == "sliding_attention" else None) * m[:, 2:3]
        x = x + attn(b + "cross_attn.", rms(x, w[b + "cross_attn_norm.weight"]), ctx, False, None)
        h = rms(x, w[b + "mlp_norm.weight"]) * (1 + m[:, 4:5]) + m[:, 3:4]
        x = x + lin(F.silu(lin(h, b + "mlp.gate_proj")) * lin(h, b + "mlp.up_proj"), b + "mlp.down_proj") * m[:, 5:6]
    m = w["scale_shift_table"] + e[:, None]
    x = rms(x, w["norm_out.weight"]) * (1 + m[:, 1:2]) + m[:, 0:1]
    v = F.conv_transpose1d(x.transpose(1, 2), w["proj_out_conv.weight"], w["proj_out_conv.bias"], stride=p)
    return v.transpose(1, 2)[:, :T]


@pytest.mark.parametrize("T", [12, 11])
def test_dit_matches_restatement(T):
    cfg = A._from_json(A.TransformerConfig, {**A.SYNTH_DIT, "attention_bias": True}, "transformer")
    w = A.random_dit_weights(cfg, 3)
    dit = A.AceStepDiT(cfg, w, "cpu")
    g = torch.Generator().manual_seed(0)
    hidden, cl, enc = torch.randn(1, T, 8, generator=g), torch.randn(1, T, 16, generator=g), torch.randn(1, 5, 32, generator=g)
    got = dit.forward(hidden, cl, 0.75, dit.embed_context(enc))
    want = _restated_dit(cfg, w, hidden, cl, 0.75, enc)
    assert got.shape == (1, T, 8)
    assert torch.allclose(got, want, atol=3e-5, rtol=1e-4)
    assert dit.forward(hidden, cl, 0.75, dit.embed_context(enc), cancel=lambda: True) is None
    # the window really bites at this length (6 tokens, window 4): widening it changes the output
    wide = A.AceStepDiT(A._from_json(A.TransformerConfig, {**A.SYNTH_DIT, "attention_bias": True, "sliding_window": 64}, "t"), w)
    assert not torch.allclose(wide.forward(hidden, cl, 0.75, wide.embed_context(enc)), got, atol=1e-6)


def test_config_cross_checks():
    from inference_b200.contracts.errors import LoadError

    vae = A._from_json(A.VaeConfig, {"audio_channels": 2, "channel_multiples": [1, 2, 4, 8, 16], "decoder_channels": 128,
                                     "decoder_input_channels": 64, "downsampling_ratios": [2, 4, 4, 6, 10],
                                     "sampling_rate": 48000}, "VAE")
    vae.validate()
    assert vae.hop_length == 1920 and vae.latents_per_second == 25.0
    for bad in ({"in_channels": 25}, {"layer_types": ["full_attention"]}, {"layer_types": ["x", "full_attention"]},
                {"num_key_value_heads": 3}, {"head_dim": 15}):
        with pytest.raises(LoadError):
            A._from_json(A.TransformerConfig, {**A.SYNTH_DIT, **bad}, "t").validate(A._from_json(A.VaeConfig, A.SYNTH_VAE, "v"))
    with pytest.raises(LoadError):
        A._from_json(A.TransformerConfig, {k: v for k, v in A.SYNTH_DIT.items() if k != "patch_size"}, "t")
    with pytest.raises(LoadError):
        A._from_json(A.VaeConfig, {**A.SYNTH_VAE, "audio_channels": 1}, "v").validate()


def test_oobleck_matches_torch_modules():
    cfg = A._from_json(A.VaeConfig, A.SYNTH_VAE, "VAE")
    sd = A.random_oobleck_weights(cfg, encoder_hidden=8, seed=5)
    wn = torch.nn.utils.weight_norm

    class Snake(torch.nn.Module):
        def __init__(self, c):
            super().__init__()
            self.alpha, self.beta = torch.nn.Parameter(torch.zeros(1, c, 1)), torch.nn.Parameter(torch.zeros(1, c, 1))

        def forward(self, x):
            return x + (self.beta.exp() + 1e-9).reciprocal() * torch.sin(self.alpha.exp() * x).pow(2)

    class Res(torch.nn.Module):
        def __init__(self, c, d):
            super().__init__()
            self.snake1, self.conv1 = Snake(c), wn(torch.nn.Conv1d(c, c, 7, dilation=d, padding=3 * d))
            self.snake2, self.conv2 = Snake(c), wn(torch.nn.Conv1d(c, c, 1))

        def forward(self, x):
            return x + self.conv2(self.snake2(self.conv1(self.snake1(x))))

    class DecBlock(torch.nn.Module):
        def __init__(self, i, o, s):
            super().__init__()
            self.snake1 = Snake(i)
            self.conv_t1 = wn(torch.nn.ConvTranspose1d(i, o, 2 * s, s, padding=math.ceil(s / 2)))
            self.res_unit1, self.res_unit2, self.res_unit3 = Res(o, 1), Res(o, 3), Res(o, 9)

        def forward(self, x):
            return self.res_unit3(self.res_unit2(self.res_unit1(self.conv_t1(self.snake1(x)))))

    class EncBlock(torch.nn.Module):
        def __init__(self, i, o, s):
            super().__init__()
            self.res_unit1, self.res_unit2, self.res_unit3 = Res(i, 1), Res(i, 3), Res(i, 9)
            self.snake1 = Snake(i)
            self.conv1 = wn(torch.nn.Conv1d(i, o, 2 * s, s, padding=math.ceil(s / 2)))

        def forward(self, x):
            return self.conv1(self.snake1(self.res_unit3(self.res_unit2(self.res_unit1(x)))))

    class Decoder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = wn(torch.nn.Conv1d(8, 16, 7, padding=3))
            self.block = torch.nn.ModuleList([DecBlock(16, 8, 4), DecBlock(8, 8, 2)])
            self.snake1, self.conv2 = Snake(8), wn(torch.nn.Conv1d(8, 2, 7, padding=3, bias=False))

        def forward(self, z):
            x = self.conv1(z)
            for b in self.block:
                x = b(x)
            return self.conv2(self.snake1(x))

    class Encoder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = wn(torch.nn.Conv1d(2, 8, 7, padding=3))
            self.block = torch.nn.ModuleList([EncBlock(8, 8, 2), EncBlock(8, 16, 4)])
            self.snake1, self.conv2 = Snake(16), wn(torch.nn.Conv1d(16, 16, 3, padding=1))

        def forward(self, x):
            x = self.conv1(x)
            for b in self.block:
                x = b(x)
            return self.conv2(self.snake1(x))

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.decoder, self.encoder = Decoder(), Encoder()

    with torch.no_grad():
        net = Net()
        net.load_state_dict(sd, strict=True)
        g = torch.Generator().manual_seed(1)
        z, wave = torch.randn(1, 8, 13, generator=g), torch.randn(1, 2, 40, generator=g) * 0.5
        want_audio, want_params = net.decoder(z), net.encoder(wave)
    vae = A.Oobleck(cfg, sd)
    got = vae.decode(z)
    assert got.shape == (1, 2, 13 * 8) and torch.allclose(got, want_audio, atol=1e-5)
    lat = vae.encode(wave)
    assert lat.shape == (1, 5, 8) and torch.allclose(lat, want_params[:, :8].transpose(1, 2), atol=1e-5)
    assert vae.decode(z, cancel=lambda: True) is None and vae.encode(wave, cancel=lambda: True) is None
    # the newer parametrisation spelling folds to the same weights
    alt = {k.replace(".weight_g", ".parametrizations.weight.original0").replace(".weight_v", ".parametrizations.weight.original1"): v
           for k, v in sd.items()}
    assert torch.allclose(A.Oobleck(cfg, alt).decode(z), got)
    from inference_b200.contracts.errors import LoadError
    with pytest.raises(LoadError):
        A.fold_weight_norm({"a.weight_g": torch.ones(1, 1, 1)})
    with pytest.raises(LoadError):
        A.Oobleck(cfg, {k: v for k, v in sd.items() if k.startswith("decoder.")}).encode(wave)


def test_scalar_quantiser():
    levels = torch.tensor([8.0, 8.0, 8.0, 5.0, 5.0, 5.0])
    g = torch.Generator().manual_seed(0)
    h = torch.randn(200, 6, generator=g) * 2.0
    q = A.fsq_round(h, levels)
    assert q.min() >= -1.0 and q.max() <= 1.0
    for lane, L in enumerate(levels.tolist()):
        grid = torch.linspace(-1.0, 1.0, int(L))
        d = (q[:, lane, None] - grid[None, :]).abs().min(dim=1).values
        assert d.max() < 1e-6                                  # every value is one of the L grid points
        assert len(torch.unique(q[:, lane])) == int(L)         # and all of them are reachable
        soft = 1.0 + 1.0 / (L - 1.0)
        c = (torch.tanh(h[:, lane] / soft) * soft).clamp(-1, 1)
        nearest = grid[(c[:, None] - grid[None, :]).abs().argmin(dim=1)]
        assert torch.allclose(q[:, lane], nearest, atol=1e-6)   # rounding to the nearest level
    assert torch.equal(A.fsq_round(torch.zeros(1, 6), levels)[0, 3:], torch.zeros(3))    # odd lanes have a level at 0


def _ramp(frames):
    f = torch.arange(frames, dtype=torch.float32)
    return torch.stack([f, -f], dim=1)


def test_stitch_rules():
    src, gen = _ramp(100), torch.full((100, 2), 9.0)
    out = A.stitch(src, gen, 100, 40, 60, 0)
    assert torch.equal(out[:40], src[:40]) and torch.equal(out[60:], src[60:]) and torch.equal(out[40:60], gen[40:60])
    assert A.crossfade_frames(40, 60) == 5 and A.crossfade_frames(0, 100) == 25
    assert A.crossfade_frames(1000, 9000) == 960 and A.crossfade_frames(10, 10) == 0
    out = A.stitch(src, gen, 100, 40, 60, 5)
    assert torch.equal(out[:40], src[:40]) and torch.equal(out[60:], src[60:])           # outside stays pristine
    assert torch.equal(out[45:55], gen[45:55])
    a = A.window_alpha(40, 60, 100, 5)
    assert a[0] < 0.25 and a[-1] < 0.25 and torch.all(a[5:15] == 1.0)
    assert abs(a[0].item() - (0.5 - 0.5 * math.cos(math.pi * 0.1))) < 1e-6
    assert torch.all(A.window_alpha(0, 60, 100, 5)[:5] == 1.0)                             # no ramp at the clip's start
    assert torch.all(A.window_alpha(40, 100, 100, 5)[-5:] == 1.0)                          # nor at its end
    # extend: the head is the source, the tail generated, frames past the source read as silence under the blend
    out = A.stitch(_ramp(50), torch.full((80, 2), 7.0), 80, 50, 80, 0)
    assert torch.equal(out[:50], _ramp(50)) and torch.all(out[50:] == 7.0)
    # a mono source is replicated to both channels
    mono = torch.arange(10, dtype=torch.float32)[:, None]
    out = A.stitch(mono, torch.full((10, 2), 3.0), 10, 4, 6, 0)
    assert torch.all(out[4:6] == 3.0) and torch.equal(out[:4, 0], out[:4, 1]) and torch.equal(out[:4, 0], mono[:4, 0])


def test_peak_normalize():
    target = 10.0 ** (-1.0 / 20.0)
    assert abs(A.peak_normalize(torch.tensor([0.5, -0.25, 0.1])).abs().max().item() - target) < 1e-6
    assert abs(A.peak_normalize(torch.tensor([3.0, -6.0])).abs().max().item() - target) < 1e-6
    assert A.peak_normalize(torch.zeros(0)).numel() == 0
    assert torch.isfinite(A.peak_normalize(torch.zeros(4))).all()


@pytest.fixture(scope="module")
def snaps(tmp_path_factory):
    root = tmp_path_factory.mktemp("acestep")
    return A.write_synthetic_snapshot(root / "turbo"), A.write_synthetic_cover_snapshot(root / "sft")


def test_edit_windows(snaps):
    from inference_b200.contracts.errors import InferenceError

    pipe = A.AceStepPipeline(snaps[0])
    lps = pipe.vae_cfg.latents_per_second                      # 6000 with the synthetic hop of 8
    assert lps == 6000.0 and pipe.latent_length(0.01) == 60
    assert pipe.edit_window("inpaint", 0.002, 0.005, 480, 60) == (60, 12, 30)
    assert pipe.edit_window("repaint", 0.002, None, 480, 60) == (60, 12, 60)
    assert pipe.edit_window("inpaint", 5.0, 6.0, 480, 60) == (60, 59, 60)          # clamped to a one-frame window
    assert pipe.edit_window("extend", 0.01, 0.02, 480, 60) == (120, 60, 120)
    assert pipe.edit_window("extend", 0.004, 0.02, 480, 60) == (120, 24, 120)
    with pytest.raises(InferenceError):
        pipe.edit_window("extend", 0.0, None, 480, 60)
    with pytest.raises(InferenceError):
        pipe.edit_window("extend", 0.0, 0.005, 480, 60)
    s = pipe.condition.src_latents(30)                                              # stored silence is 12 frames: tiled
    assert s.shape == (1, 30, 8) and torch.equal(s[:, 12:24], s[:, :12])
    ctx = pipe.encode_context("a red fox", "the quick brown fox", A.Metadata(bpm=120.0))
    plain = pipe.encode_context("a red fox", "", A.Metadata(bpm=120.0))
    assert ctx.shape[2] == 32 and ctx.shape[1] > plain.shape[1] and plain.shape[1] >= 2
    assert pipe.encode_context("", "", A.Metadata()).shape == (1, 2, 32)           # zero text row + the timbre token


def test_generator_conformance_edits_and_cover(snaps, monkeypatch):
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.errors import InferenceError, LoadError, Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams, Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import AudioTrack
    from inference_b200.contracts.gen_core.runtime import WeightsSource
    from inference_b200.testkit.audio_generator import AudioProfile, audio_conformance

    turbo, sft = snaps
    reg = provider_registry("cpu")
    assert "cpu_acestep_v15_turbo" in reg.ids()
    gen = reg.load("cpu_acestep_v15_turbo", LoadSpec.from_dir(turbo))
    d = gen.descriptor()
    assert d.family == "acestep" and not d.capabilities.supports_negative_prompt and not d.capabilities.supports_guidance
    assert d.capabilities.audio_edit_modes == ["inpaint", "repaint", "extend", "cover"]
    assert d.capabilities.audio_sample_rates == [48_000] and d.capabilities.max_audio_duration_secs == 600.0
    monkeypatch.setattr(A, "DEFAULT_SECONDS", 0.01)
    monkeypatch.setattr(A, "DEFAULT_STEPS", 2)
    monkeypatch.setattr(A, "COVER_STEPS", 2)
    audio_conformance(gen, AudioProfile(prompt="upbeat electronic dance track"))
    out = gen.generate(GenerationRequest(prompt="calm piano", seed=3, audio=AudioParams(target_duration=0.1205, lyrics="la la",
                                                                                       bpm=90.0, musical_key="C minor", language="en")))
    t = out.audio
    assert t.channels == 2 and len(t.samples) == 2 * round(48000 * 0.1205)
    assert abs(max(abs(x) for x in t.samples) - 10.0 ** (-1 / 20)) < 1e-5

    # ---- region edits ----
    frames = 480
    g = torch.Generator().manual_seed(9)
    src = (torch.randn(frames, 2, generator=g) * 0.2)
    track = AudioTrack(48_000, 2, src.reshape(-1).tolist())

    def edit_req(mode, region, **kw):
        return GenerationRequest(prompt="calm piano", seed=3, audio=AudioParams(), **{"steps": 2, **kw},
                                 conditioning=[Conditioning(ConditioningKind.AUDIO_EDIT, audio=track, mode=mode, region=region)])

    got = torch.tensor(gen.generate(edit_req("inpaint", (0.0025, 0.0075))).audio.samples).view(-1, 2)
    f0, f1 = 15 * 8, 45 * 8
    assert got.shape == (frames, 2)
    assert torch.equal(got[:f0], src[:f0]) and torch.equal(got[f1:], src[f1:])        # untouched outside, bit for bit
    assert not torch.allclose(got[f0 + 60: f1 - 60], src[f0 + 60: f1 - 60], atol=1e-3)
    ext = torch.tensor(gen.generate(edit_req("extend", (0.01, 0.015))).audio.samples).view(-1, 2)
    assert ext.shape == (720, 2) and torch.equal(ext[:frames], src) and ext[frames + 40:].abs().max() > 0
    mono = AudioTrack(48_000, 1, src[:, 0].tolist())
    r = GenerationRequest(prompt="calm piano", seed=3, steps=2, audio=AudioParams(),
                          conditioning=[Conditioning(ConditioningKind.AUDIO_EDIT, audio=mono, mode="repaint", region=(0.005, None))])
    rp = torch.tensor(gen.generate(r).audio.samples).view(-1, 2)
    assert torch.equal(rp[:240, 0], src[:240, 0]) and torch.equal(rp[:240, 1], src[:240, 0])

    # ---- request validation ----
    for bad in (edit_req("inpaint", None), edit_req("inpaint", (0.02, None)), edit_req("inpaint", (0.0, 0.5)),
                edit_req("extend", (0.0, None)), edit_req("extend", (0.0, 0.005)), edit_req("inpaint", (0.0, 0.005), steps=201),
                edit_req("inpaint", (0.0, 0.005), scheduler_shift=0.0)):
        with pytest.raises(InferenceError):
            gen.validate(bad)
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt="x", audio=AudioParams(target_duration=0.01)))
    low = AudioTrack(44_100, 2, [0.0] * 200)
    with pytest.raises(Unsupported):
        gen.validate(GenerationRequest(prompt="x", audio=AudioParams(), conditioning=[
            Conditioning(ConditioningKind.AUDIO_EDIT, audio=low, mode="inpaint", region=(0.0, 0.001))]))
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt="x", audio=AudioParams(), conditioning=[
            Conditioning(ConditioningKind.AUDIO_EDIT, audio=AudioTrack(48_000, 2, []), mode="inpaint", region=(0.0, 0.001))]))

    # ---- cover: needs the staged fine-tuned snapshot ----
    with pytest.raises(InferenceError, match="sft_cover"):
        gen.generate(edit_req("cover", None))
    spec = LoadSpec.from_dir(turbo)
    spec.components["sft_cover"] = WeightsSource.dir(sft)
    cgen = reg.load("cpu_acestep_v15_turbo", spec)
    events = []
    cov = torch.tensor(cgen.generate(edit_req("cover", None), events.append).audio.samples).view(-1, 2)
    assert cov.shape == (frames, 2) and torch.isfinite(cov).all() and not torch.allclose(cov, src, atol=1e-3)
    mods, _ = cgen.pipeline().cover_modules(sft)
    lat = torch.randn(1, 13, 8, generator=g)
    tokens = mods.tokenize(lat, cgen.pipeline().condition.src_latents(5))
    assert tokens.shape == (1, 3, 32) and mods.detokenize(tokens).shape == (1, 15, 8)

    # ---- load errors ----
    bad = LoadSpec.from_dir(turbo)
    bad.components["sft_cover"] = WeightsSource.file(sft / "transformer" / "diffusion_pytorch_model.safetensors")
    with pytest.raises(LoadError):
        reg.load("cpu_acestep_v15_turbo", bad)
    unknown = LoadSpec.from_dir(turbo)
    unknown.components["vocoder"] = WeightsSource.dir(sft)
    with pytest.raises(LoadError):
        reg.load("cpu_acestep_v15_turbo", unknown)
    with pytest.raises(LoadError):
        reg.load("cpu_acestep_v15_turbo", LoadSpec(weights=WeightsSource.file(turbo / "model_index.json")))
    empty = turbo.parent / "empty"
    empty.mkdir()
    with pytest.raises(LoadError):
        reg.load("cpu_acestep_v15_turbo", LoadSpec.from_dir(empty)).generate(GenerationRequest(prompt="x"))
