"""MOSS-SoundEffect: prompt text rules, the shifted flow schedule, the DiT against an independent module-style
restatement, the DAC decoder against torch.nn layers with weight norm, and the audio-generator conformance suite."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.audio import moss_sfx as M


def test_prompt_text_rules():
    assert M.with_duration_suffix("glass shattering", 4.0) == "glass shattering duration: 4.0s"
    assert M.with_duration_suffix("  rain on a tin roof \n", M.round_seconds(12.34)) == "rain on a tin roof duration: 12.3s"
    assert M.clean_prompt("a   dog\n\tbarks") == "a dog barks"
    assert M.clean_prompt("thunder &amp; rain") == "thunder & rain"
    assert M.clean_prompt("&amp;amp;") == "&"
    assert M.clean_prompt("&#65;&#x42;") == "AB"
    assert M.clean_prompt("   ") == ""
    assert M.clean_prompt("AT&T &unknown; x") == "AT&T &unknown; x"


def test_schedule():
    cfg = M.SchedulerConfig(5.0, 0.0, True, 1000)
    s = M.flow_sigmas(cfg, 4)
    for got, want in zip(s, [1.0, 0.9375, 5.0 * 0.5 / 3.0, 0.625, 0.0]):
        assert abs(got - want) < 1e-12
    assert abs(M.flow_sigmas(cfg, 4, 1.0)[1] - 0.75) < 1e-12
    plain = M.flow_sigmas(M.SchedulerConfig(1.0, 0.25, False, 1000), 4)
    assert plain == pytest.approx([1.0, 0.75, 0.5, 0.25, 0.0])


def _restated_dit(cfg, w, lat, timestep, context):
    """Module-by-module restatement with torch.nn.functional only (heads-first layout, explicit softmax)."""
    lin = lambda x, p: F.linear(x, w[p + ".weight"], w.get(p + ".bias"))      # noqa: E731
    H, D = cfg.num_heads, cfg.dim // cfg.num_heads
    half = cfg.freq_dim // 2
    ang = timestep * torch.pow(10000.0, -torch.arange(half, dtype=torch.float64) / half)
    t_emb = torch.cat([ang.cos(), ang.sin()]).float()[None]
    ce = "condition_embedder."
    t = lin(F.silu(lin(t_emb, ce + "time_embedder.linear_1")), ce + "time_embedder.linear_2")
    t_mod = lin(F.silu(t), ce + "time_proj").view(1, 6, cfg.dim)
    ctx = lin(F.gelu(lin(context, ce + "text_embedder.linear_1"), approximate="tanh"), ce + "text_embedder.linear_2")
    x = F.conv1d(lat, w["patch_embedding.weight"], w["patch_embedding.bias"]).transpose(1, 2)
    T = x.shape[1]
    rms = lambda v, g: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * g       # noqa: E731
    heads = lambda v: v.view(1, -1, H, D).transpose(1, 2)                                   # noqa: E731
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    th = (torch.arange(T, dtype=torch.float64)[:, None] * inv).float()

    def rope(v):                           # [1, H, T, D], adjacent pairs
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * th.cos() - b * th.sin(), a * th.sin() + b * th.cos()], -1).flatten(-2)

    def attn(q, k, v):
        p = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(D), -1)
        return (p @ v).transpose(1, 2).reshape(1, -1, H * D)

    ln = lambda v: F.layer_norm(v, (cfg.dim,), eps=cfg.eps)                                  # noqa: E731
    for i in range(cfg.num_layers):
        p = f"blocks.{i}."
        m = w[p + "scale_shift_table"] + t_mod
        h = ln(x) * (1 + m[:, 1:2]) + m[:, 0:1]
        q = rope(heads(rms(lin(h, p + "attn1.to_q"), w[p + "attn1.norm_q.weight"])))
        k = rope(heads(rms(lin(h, p + "attn1.to_k"), w[p + "attn1.norm_k.weight"])))
        x = x + lin(attn(q, k, heads(lin(h, p + "attn1.to_v"))), p + "attn1.to_out.0") * m[:, 2:3]
        h = F.layer_norm(x, (cfg.dim,), w[p + "norm2.weight"], w[p + "norm2.bias"], cfg.eps)
        q = heads(rms(lin(h, p + "attn2.to_q"), w[p + "attn2.norm_q.weight"]))
        k = heads(rms(lin(ctx, p + "attn2.to_k"), w[p + "attn2.norm_k.weight"]))
        x = x + lin(attn(q, k, heads(lin(ctx, p + "attn2.to_v"))), p + "attn2.to_out.0")
        h = ln(x) * (1 + m[:, 4:5]) + m[:, 3:4]
        x = x + lin(F.gelu(lin(h, p + "ffn.net.0.proj"), approximate="tanh"), p + "ffn.net.2") * m[:, 5:6]
    m = w["scale_shift_table"] + t[:, None]
    return lin(ln(x) * (1 + m[:, 1:2]) + m[:, 0:1], "proj_out").transpose(1, 2)


def test_dit_matches_restatement():
    cfg = M.DitConfig(in_dim=8, out_dim=8, text_dim=12, freq_dim=16, dim=32, ffn_dim=48, num_heads=4, num_layers=2)
    w = M.random_dit_weights(cfg, 3)
    dit = M.SfxDiT(cfg, w, "cpu")
    torch.manual_seed(0)
    lat, ctx = torch.randn(1, 8, 11), torch.randn(1, 7, 12)
    cos, sin = M.rope_tables(8, 11, "cpu")
    got = dit.forward(lat, 937.5, dit.embed_context(ctx), cos, sin)
    want = _restated_dit(cfg, w, lat, 937.5, ctx)
    assert got.shape == (1, 8, 11)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)
    assert dit.forward(lat, 937.5, dit.embed_context(ctx), cos, sin, cancel=lambda: True) is None


def test_dac_decoder_matches_torch_modules():
    rates, dim, latent = (3, 2), 8, 4
    sd = M.random_dac_weights(dim, rates, latent, seed=5)
    wn = torch.nn.utils.weight_norm

    class Snake(torch.nn.Module):
        def __init__(self, c):
            super().__init__()
            self.alpha = torch.nn.Parameter(torch.ones(1, c, 1))

        def forward(self, x):
            return x + (self.alpha + 1e-9).reciprocal() * torch.sin(self.alpha * x).pow(2)

    def unit(c, d):
        class U(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.block = torch.nn.Sequential(Snake(c), wn(torch.nn.Conv1d(c, c, 7, dilation=d, padding=3 * d)), Snake(c),
                                                 wn(torch.nn.Conv1d(c, c, 1)))

            def forward(self, x):
                return x + self.block(x)
        return U()

    def block(c, r):
        class B(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.block = torch.nn.Sequential(
                    Snake(c), wn(torch.nn.ConvTranspose1d(c, c // 2, 2 * r, r, padding=math.ceil(r / 2), output_padding=r % 2)),
                    unit(c // 2, 1), unit(c // 2, 3), unit(c // 2, 9))

            def forward(self, x):
                return self.block(x)
        return B()

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.post_quant_conv = torch.nn.Conv1d(latent, latent, 1)
            layers, c = [wn(torch.nn.Conv1d(latent, dim, 7, padding=3))], dim
            for r in rates:
                layers.append(block(c, r))
                c //= 2
            layers += [Snake(c), wn(torch.nn.Conv1d(c, 1, 7, padding=3)), torch.nn.Tanh()]
            self.decoder = torch.nn.Module()
            self.decoder.model = torch.nn.Sequential(*layers)

        def forward(self, z):
            return self.decoder.model(self.post_quant_conv(z))

    with torch.no_grad():
        net = Net()
        missing = net.load_state_dict(sd, strict=True)
        assert not missing.missing_keys
        z = torch.randn(1, latent, 13, generator=torch.Generator().manual_seed(1))
        want = net(z)
    got = M.DacDecoder(sd, "cpu", rates).decode(z)
    assert got.shape == (1, 1, 13 * 6)
    assert torch.allclose(got, want, atol=1e-5)


def test_generator_conformance_and_length_law(tmp_path):
    from inference_b200.audio.catalog import provider_registry
    from inference_b200.contracts.errors import InferenceError, LoadError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import AudioParams
    from inference_b200.testkit.audio_generator import AudioProfile, audio_conformance

    snap = M.write_synthetic_snapshot(tmp_path / "sfx", sample_rate=4800)      # 5 latent frames per second keeps it quick
    reg = provider_registry("cpu")
    assert "cpu_moss_sfx_v2" in reg.ids()
    gen = reg.load("cpu_moss_sfx_v2", LoadSpec.from_dir(snap))
    d = gen.descriptor()
    assert d.family == "moss_soundeffect" and d.capabilities.supports_negative_prompt and d.capabilities.supports_guidance
    assert d.capabilities.audio_sample_rates == [48_000] and d.capabilities.max_audio_duration_secs == 30.0

    # the conformance run uses few steps through the request the suite builds: patch the default down
    old = M.DEFAULT_STEPS
    M.DEFAULT_STEPS = 3
    try:
        audio_conformance(gen, AudioProfile(prompt="glass shattering on a stone floor", target_duration=1.3))
    finally:
        M.DEFAULT_STEPS = old
    pipe = gen.pipeline()
    assert pipe.window_seconds(0.4) == 1 and pipe.window_seconds(12.2) == 13 and pipe.window_seconds(99.0) == 30
    out = pipe.synthesize("rain", 1.26, 2, 1.0, "", 5)
    assert out.numel() == round(4800 * 1.3)
    guided = pipe.synthesize("rain", 1.26, 2, 4.0, "hiss", 5)
    assert guided.shape == out.shape and not torch.allclose(guided, out)
    for bad in (dict(steps=1001), dict(guidance=0.5), dict(guidance=25.0), dict(scheduler_shift=0.0)):
        with pytest.raises(InferenceError):
            gen.validate(GenerationRequest(prompt="rain", audio=AudioParams(), **bad))
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(prompt="rain", audio=AudioParams(target_duration=0.04)))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(LoadError):
        reg.load("cpu_moss_sfx_v2", LoadSpec.from_dir(empty)).generate(GenerationRequest(prompt="rain"))
