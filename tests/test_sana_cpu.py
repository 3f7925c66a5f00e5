"""SANA: linear attention against its quadratic form, the trunk against an independent restatement, the DC-AE decoder
against torch.nn modules carrying the same weights, the consistency sampler's algebra, provider conformance."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_sana as S

CFG = S.SanaConfig(num_attention_heads=2, attention_head_dim=8, num_layers=2, num_cross_attention_heads=2,
                   cross_attention_head_dim=8, caption_channels=12, in_channels=4, out_channels=4, guidance_embeds=True,
                   qk_norm=True)


def test_relu_linear_attention_equals_the_quadratic_form():
    torch.manual_seed(0)
    q, k, v = torch.rand(2, 3, 8, 10), torch.rand(2, 3, 8, 10), torch.randn(2, 3, 8, 10)
    got = S.relu_linear_attention(q, k, v, 1e-15)
    scores = torch.einsum("bgdn,bgdm->bgnm", q, k)                     # query n, key m
    want = torch.einsum("bgnm,bgdm->bgdn", scores / scores.sum(-1, keepdim=True), v)
    assert torch.allclose(got, want, atol=1e-5)


def _direct(w, cfg, latent, cap, t, g):
    D = cfg.inner
    lin = lambda x, n: x @ w[n + ".weight"].t() + (w[n + ".bias"] if n + ".bias" in w else 0)      # noqa: E731
    ln = lambda x: F.layer_norm(x, (D,), eps=cfg.norm_eps)              # noqa: E731
    rms = lambda x, k, e: x / torch.sqrt((x * x).mean(-1, keepdim=True) + e) * w[k]                # noqa: E731

    def temb(s, name):
        f = torch.exp(-math.log(10000.0) * torch.arange(128).float() / 128)
        e = torch.cat([torch.cos(s * f), torch.sin(s * f)])
        return lin(F.silu(lin(e, name + ".linear_1")), name + ".linear_2")

    C, H, W = latent.shape
    x = torch.stack([lin(latent[:, i, j], "patch_embed.proj.flat") for i in range(H) for j in range(W)])
    emb = temb(t, "time_embed.timestep_embedder") + temb(g, "time_embed.guidance_embedder")
    tm = lin(F.silu(emb), "time_embed.linear").view(6, D)
    c = rms(lin(F.gelu(lin(cap, "caption_projection.linear_1"), approximate="tanh"), "caption_projection.linear_2"),
            "caption_norm.weight", cfg.caption_norm_eps)
    for i in range(cfg.num_layers):
        b = f"transformer_blocks.{i}"
        m = w[b + ".scale_shift_table"] + tm
        h = ln(x) * (1 + m[1]) + m[0]
        a = b + ".attn1."
        q = rms(lin(h, a + "to_q"), a + "norm_q.weight", 1e-5).view(-1, cfg.num_attention_heads, cfg.attention_head_dim).relu()
        k = rms(lin(h, a + "to_k"), a + "norm_k.weight", 1e-5).view(-1, cfg.num_attention_heads, cfg.attention_head_dim).relu()
        v = lin(h, a + "to_v").view(-1, cfg.num_attention_heads, cfg.attention_head_dim)
        s = torch.einsum("nhd,mhd->hnm", q, k)
        o = torch.einsum("hnm,mhd->nhd", s / (s.sum(-1, keepdim=True) + cfg.attn_eps), v).reshape(-1, D)
        x = x + m[2] * lin(o, a + "to_out.0")
        a = b + ".attn2."
        hd = cfg.cross_attention_head_dim
        q = rms(lin(x, a + "to_q"), a + "norm_q.weight", 1e-5).view(-1, cfg.num_cross_attention_heads, hd)
        k = rms(lin(c, a + "to_k"), a + "norm_k.weight", 1e-5).view(-1, cfg.num_cross_attention_heads, hd)
        v = lin(c, a + "to_v").view(-1, cfg.num_cross_attention_heads, hd)
        s = (torch.einsum("nhd,mhd->hnm", q, k) / math.sqrt(hd)).softmax(-1)
        x = x + lin(torch.einsum("hnm,mhd->nhd", s, v).reshape(-1, D), a + "to_out.0")
        h = (ln(x) * (1 + m[4]) + m[3]).view(H, W, D).permute(2, 0, 1)[None]
        f = F.silu(F.conv2d(h, w[b + ".ff.conv_inverted.weight"], w[b + ".ff.conv_inverted.bias"]))
        f = F.conv2d(f, w[b + ".ff.conv_depth.weight"], w[b + ".ff.conv_depth.bias"], padding=1, groups=f.shape[1])
        hid = cfg.ffn_hidden
        f = F.conv2d(f[:, :hid] * F.silu(f[:, hid:]), w[b + ".ff.conv_point.weight"])
        x = x + m[5] * f[0].permute(1, 2, 0).reshape(-1, D)
    fm = w["scale_shift_table"] + emb
    out = lin(ln(x) * (1 + fm[1]) + fm[0], "proj_out")
    return out.view(H, W, cfg.out_channels).permute(2, 0, 1)


def test_trunk_matches_restatement():
    torch.manual_seed(2)
    w = S.random_sana_weights(CFG, seed=5, std=0.2)
    model = S.SanaDiT(CFG, w)
    latent, cap = torch.randn(1, 4, 3, 5), torch.randn(1, 7, 12)
    t, g = torch.tensor([412.0]), torch.tensor([0.45])
    got = model.forward(latent, cap, t, g)
    w2 = dict(w)
    w2["patch_embed.proj.flat.weight"], w2["patch_embed.proj.flat.bias"] = w["patch_embed.proj.weight"].reshape(CFG.inner, -1), w["patch_embed.proj.bias"]
    want = _direct(w2, CFG, latent[0], cap[0], t[0], g[0])
    assert torch.allclose(got[0], want, atol=2e-4, rtol=1e-3), (got[0] - want).abs().max()
    pre = model.caption(cap)
    assert torch.allclose(model.forward(latent, pre, t, g, projected=True), got, atol=1e-6)


def test_dcae_decoder_matches_module_restatement():
    cfg = S.DcAeConfig(latent_channels=4, attention_head_dim=4, block_out_channels=(8, 8, 16), layers_per_block=(1, 1, 2),
                       block_types=("res", "res", "evit"), qkv_multiscales=(3,))
    w = S.random_dcae_weights(cfg, seed=3)
    dec = S.DcAeDecoder(cfg, w)
    z = torch.randn(1, 4, 2, 3)
    got = dec.decode(z)
    assert got.shape == (1, 3, 8, 12)

    def trms(x, p):
        return x / torch.sqrt(x.pow(2).mean(1, keepdim=True) + 1e-5) * w[p + ".weight"].view(1, -1, 1, 1) + w[p + ".bias"].view(1, -1, 1, 1)

    def conv(x, p, **kw):
        return F.conv2d(x, w[p + ".weight"], w.get(p + ".bias"), **kw)

    def res(x, p):
        return trms(conv(F.silu(conv(x, p + ".conv1", padding=1)), p + ".conv2", padding=1), p + ".norm") + x

    def evit(x, p):
        B, C, H, W = x.shape
        hd, heads = 4, C // 4
        lin1 = lambda n: F.conv2d(x, w[f"{p}.attn.{n}.weight"].view(C, C, 1, 1))      # noqa: E731
        qkv = torch.cat([lin1("to_q"), lin1("to_k"), lin1("to_v")], 1)
        ms = conv(conv(qkv, p + ".attn.to_qkv_multiscale.0.proj_in", padding=1, groups=3 * C),
                  p + ".attn.to_qkv_multiscale.0.proj_out", groups=3 * heads)
        hid = torch.cat([qkv, ms], 1).view(B, 2 * heads, 3 * hd, H * W)
        q, k, v = hid[:, :, :hd].relu(), hid[:, :, hd:2 * hd].relu(), hid[:, :, 2 * hd:]
        s = torch.einsum("bgdn,bgdm->bgnm", q, k)
        o = torch.einsum("bgnm,bgdm->bgdn", s / (s.sum(-1, keepdim=True) + 1e-15), v).reshape(B, 2 * C, H, W)
        x = trms(F.conv2d(o, w[p + ".attn.to_out.weight"].view(C, 2 * C, 1, 1)), p + ".attn.norm_out") + x
        c = p + ".conv_out"
        f = conv(F.silu(conv(x, c + ".conv_inverted")), c + ".conv_depth", padding=1, groups=8 * C)
        f = conv(f[:, :4 * C] * F.silu(f[:, 4 * C:]), c + ".conv_point")
        return trms(f, c + ".norm") + x

    def up(x, p, out_ch):
        y = conv(F.interpolate(x, scale_factor=2.0, mode="nearest"), p + ".conv", padding=1)
        B, C, H, W = x.shape
        r = out_ch * 4 // C
        rep = x[:, :, None].expand(B, C, r, H, W).reshape(B, C * r, H, W)
        return y + F.pixel_shuffle(rep, 2)

    h = conv(z, "decoder.conv_in", padding=1) + z[:, :, None].expand(1, 4, 4, 2, 3).reshape(1, 16, 2, 3)
    h = evit(evit(h, "decoder.up_blocks.2.0"), "decoder.up_blocks.2.1")
    h = res(up(h, "decoder.up_blocks.1.0", 8), "decoder.up_blocks.1.1")
    h = res(up(h, "decoder.up_blocks.0.0", 8), "decoder.up_blocks.0.1")
    want = conv(F.relu(trms(h, "decoder.norm_out")), "decoder.conv_out", padding=1)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4), (got - want).abs().max()


def test_scm_sampler_algebra():
    from inference_b200.contracts.gen_core.sampling import ScmScheduler, TorchLatentOps, run_scm_sampler

    s2 = ScmScheduler.new(2)
    assert s2.timesteps == [math.pi / 2, 1.3, 0.0] and s2.num_steps == 2
    s4 = ScmScheduler.new(4)
    assert len(s4.timesteps) == 5 and abs(s4.timesteps[1] - math.pi / 2 * 0.75) < 1e-9 and s4.timesteps[-1] == 0.0
    assert abs(s2.scm_timestep(0) - 1.0) < 1e-6 and abs(s2.input_scale(0) - 1.0) < 1e-6      # t = pi / 2: pure noise
    # an exact flow-velocity oracle: x_t = (1 - tau) x0 + tau z, v = z - x0; the sampler must return x0 in one step
    x0 = torch.tensor([0.3, -0.7, 1.1])
    noise = torch.tensor([0.5, -1.5, 0.25])

    def predict(x_in, tau):
        assert abs(tau - 1.0) < 1e-6 and torch.allclose(x_in, noise, atol=1e-6)
        return noise - x0 / 0.5                                         # flow velocity in sigma_data-normalised units

    out = run_scm_sampler(TorchLatentOps(), ScmScheduler.new(1), noise, 0, predict)
    assert torch.allclose(out, x0 / 0.5, atol=1e-5)
    # re-noising between steps uses the seeded, step-indexed generator: same seed -> same path
    f = lambda x_in, tau: x_in * 0.1                                     # noqa: E731
    a = run_scm_sampler(TorchLatentOps(), s2, noise, 7, f)
    b = run_scm_sampler(TorchLatentOps(), s2, noise, 7, f)
    c = run_scm_sampler(TorchLatentOps(), s2, noise, 8, f)
    assert torch.equal(a, b) and not torch.equal(a, c)


def test_sana_providers_conform(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.sana import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "sana")
    reg = provider_registry("cpu")
    assert sorted(i for i in reg.ids() if "sana" in i) == ["cpu_sana_1600m", "cpu_sana_sprint_1600m"]
    assert reg.descriptor_conformance_errors() == []
    base = reg.load("cpu_sana_1600m", LoadSpec.from_dir(snap))
    kit.conformance(base, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_sana_1600m", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = base.generate(GenerationRequest(**req, guidance=1.0)).images[0].pixels
    b = base.generate(GenerationRequest(**req)).images[0].pixels
    c = base.generate(GenerationRequest(**req, guidance=4.5, negative_prompt="")).images[0].pixels
    assert a != b and b == c and len(a) == 256 * 256 * 3
    sprint = reg.load("cpu_sana_sprint_1600m", LoadSpec.from_dir(snap))
    kit.conformance(sprint, kit.Profile(steps=2, cancel_steps=4))
    s1 = sprint.generate(GenerationRequest(**req)).images[0].pixels
    s2 = sprint.generate(GenerationRequest(**req, guidance=2.0)).images[0].pixels
    assert s1 != s2 and len(s1) == 256 * 256 * 3
    with pytest.raises(InferenceError):
        sprint.generate(GenerationRequest(**req, negative_prompt="blurry"))
    with pytest.raises(InferenceError):
        sprint.generate(GenerationRequest(**req, sampler="heun"))
