"""FLUX.2: the MMDiT against an independent restatement (complex rotary over four axes, explicit softmax attention,
shared modulation), token / latent layout helpers, the schedule's documented properties, and provider conformance."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_flux2 as X

CFG = X.Flux2Config(num_double_layers=2, num_single_layers=2, num_heads=2, head_dim=16, in_channels=12, out_channels=12,
                    joint_attention_dim=20, axes_dim=(4, 4, 4, 4), guidance_embed=True)


def _direct(w, cfg, hidden, context, img_ids, txt_ids, t, g):
    D, nh, hd = cfg.inner, cfg.num_heads, cfg.head_dim
    lin = lambda x, n: x @ w[n + ".weight"].t()                      # noqa: E731
    ln = lambda x: F.layer_norm(x, (x.shape[-1],), eps=1e-6)         # noqa: E731

    def emb(s, name):
        half = cfg.timestep_channels // 2
        f = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
        e = torch.cat([torch.cos(s * f), torch.sin(s * f)])
        return lin(F.silu(lin(e, name + ".linear_1")), name + ".linear_2")

    temb = emb(t, "time_guidance_embed.timestep_embedder") + emb(g * 1000.0, "time_guidance_embed.guidance_embedder")
    ids = torch.cat([txt_ids, img_ids]).double()
    ang = torch.cat([ids[:, a:a + 1] * (1.0 / cfg.rope_theta ** (torch.arange(0, d, 2).double() / d))
                     for a, d in enumerate(cfg.axes_dim)], -1)
    fr = torch.polar(torch.ones_like(ang), ang)

    def rot(x):
        xc = torch.view_as_complex(x.double().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * fr[:, None, :]).flatten(-2).float()

    def rms(x, key):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w[key]

    def attn(q, k, v):
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        return torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(q.shape[0], D)

    def sets(name, n):
        m = lin(F.silu(temb), name + ".linear").chunk(3 * n)
        return [(m[3 * i], m[3 * i + 1], m[3 * i + 2]) for i in range(n)]

    def glu(x):
        a, b = x.chunk(2, -1)
        return F.silu(a) * b

    img, txt = lin(hidden, "x_embedder"), lin(context, "context_embedder")
    im, tm = sets("double_stream_modulation_img", 2), sets("double_stream_modulation_txt", 2)
    nt = txt.shape[0]
    for i in range(cfg.num_double_layers):
        p = f"transformer_blocks.{i}"
        a = p + ".attn."
        ni, ntx = ln(img) * (1 + im[0][1]) + im[0][0], ln(txt) * (1 + tm[0][1]) + tm[0][0]
        q = torch.cat([rms(lin(ntx, a + "add_q_proj").view(-1, nh, hd), a + "norm_added_q.weight"),
                       rms(lin(ni, a + "to_q").view(-1, nh, hd), a + "norm_q.weight")])
        k = torch.cat([rms(lin(ntx, a + "add_k_proj").view(-1, nh, hd), a + "norm_added_k.weight"),
                       rms(lin(ni, a + "to_k").view(-1, nh, hd), a + "norm_k.weight")])
        v = torch.cat([lin(ntx, a + "add_v_proj").view(-1, nh, hd), lin(ni, a + "to_v").view(-1, nh, hd)])
        o = attn(rot(q), rot(k), v)
        img = img + im[0][2] * lin(o[nt:], a + "to_out.0")
        txt = txt + tm[0][2] * lin(o[:nt], a + "to_add_out")
        img = img + im[1][2] * lin(glu(lin(ln(img) * (1 + im[1][1]) + im[1][0], p + ".ff.linear_in")), p + ".ff.linear_out")
        txt = txt + tm[1][2] * lin(glu(lin(ln(txt) * (1 + tm[1][1]) + tm[1][0], p + ".ff_context.linear_in")),
                                   p + ".ff_context.linear_out")
    x = torch.cat([txt, img])
    (sh, sc, gt), = sets("single_stream_modulation", 1)
    for i in range(cfg.num_single_layers):
        a = f"single_transformer_blocks.{i}.attn."
        pr = lin(ln(x) * (1 + sc) + sh, a + "to_qkv_mlp_proj")
        q, k, v, mlp = pr[:, :D], pr[:, D:2 * D], pr[:, 2 * D:3 * D], pr[:, 3 * D:]
        o = attn(rot(rms(q.reshape(-1, nh, hd), a + "norm_q.weight")), rot(rms(k.reshape(-1, nh, hd), a + "norm_k.weight")),
                 v.reshape(-1, nh, hd))
        x = x + gt * lin(torch.cat([o, glu(mlp)], -1), a + "to_out")
    s2 = lin(F.silu(temb), "norm_out.linear")
    return lin(ln(x[nt:]) * (1 + s2[:D]) + s2[D:], "proj_out")


def test_dit_matches_restatement():
    torch.manual_seed(1)
    w = X.random_flux2_weights(CFG, seed=2, std=0.2)
    model = X.Flux2DiT(CFG, w)
    h, wd, L = 3, 4, 5
    hidden, ctx = torch.randn(1, h * wd, 12), torch.randn(1, L, 20)
    img_ids, txt_ids = X.grid_ids(h, wd), X.text_ids(L)
    t, g = torch.tensor([630.0]), torch.tensor([3.5])
    got = model.forward(hidden, ctx, img_ids, txt_ids, t, g)
    want = _direct(w, CFG, hidden[0], ctx[0], img_ids, txt_ids, t[0], g[0])
    assert got.shape == (1, 12, 12) and torch.allclose(got[0], want, atol=2e-4, rtol=1e-3), (got[0] - want).abs().max()
    no_g = model.forward(hidden, ctx, img_ids, txt_ids, t, None)
    assert not torch.allclose(no_g, got, atol=1e-4)


def test_ids_and_latent_layouts():
    ids = X.grid_ids(2, 3)
    assert ids.tolist() == [[0, 0, 0, 0], [0, 0, 1, 0], [0, 0, 2, 0], [0, 1, 0, 0], [0, 1, 1, 0], [0, 1, 2, 0]]
    assert X.grid_ids(2, 2, 10)[:, 0].tolist() == [10.0] * 4
    assert X.text_ids(4).tolist() == [[0, 0, 0, 0], [0, 0, 0, 1], [0, 0, 0, 2], [0, 0, 0, 3]]
    x = torch.arange(8.0).view(1, 8, 1, 1)                    # channel value = c * 4 + ph * 2 + pw
    u = X.vae_unpatchify(x)
    assert u.shape == (1, 2, 2, 2) and u[0, 0].tolist() == [[0, 1], [2, 3]] and u[0, 1].tolist() == [[4, 5], [6, 7]]
    y = torch.randn(2, 3, 4, 6)
    assert torch.equal(X.vae_unpatchify(X.vae_patchify(y)), y)
    full = X.Flux2Config.klein_9b()
    assert full.inner == 4096 and full.mlp_hidden == 12288 and sum(full.axes_dim) == full.head_dim
    dev = X.Flux2Config.dev()
    assert dev.inner == 6144 and dev.num_single_layers == 48 and dev.joint_attention_dim == 15360


def test_schedule_properties():
    from inference_b200.media import flux2 as P

    s = P.build_sigmas(4, P.compute_mu(4096, 4))
    assert len(s) == 5 and 0.0 < s[0] <= 1.0 and s[-1] == 0.0 and all(a > b for a, b in zip(s, s[1:]))
    assert abs(P.compute_mu(5000, 4) - P.compute_mu(5000, 50)) < 1e-9        # above 4300 tokens mu ignores the step count
    assert abs(P.compute_mu(5000, 4) - (0.00016927 * 5000 + 0.45666666)) < 1e-9
    m10 = 8.73809524e-5 * 1024 + 1.89833333
    m200 = 0.00016927 * 1024 + 0.45666666
    assert abs(P.compute_mu(1024, 10) - m10) < 1e-6 and abs(P.compute_mu(1024, 200) - m200) < 1e-6
    assert P.build_sigmas(1, 0.7) == [1.0, 0.0]


def test_flux2_providers_conform(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.flux2 import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "f2")
    reg = provider_registry("cpu")
    assert sorted(i for i in reg.ids() if "flux2" in i) == ["cpu_flux2_dev", "cpu_flux2_klein_9b"]
    assert reg.descriptor_conformance_errors() == []
    klein = reg.load("cpu_flux2_klein_9b", LoadSpec.from_dir(snap))
    kit.conformance(klein, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_flux2_klein_9b", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = klein.generate(GenerationRequest(**req)).images[0].pixels                       # guidance 1: one forward
    b = klein.generate(GenerationRequest(**req, guidance=3.0)).images[0].pixels          # negative pass, prompt " "
    c = klein.generate(GenerationRequest(**req, guidance=3.0, negative_prompt=" ")).images[0].pixels
    assert a != b and b == c and len(a) == 256 * 256 * 3
    dev = reg.load("cpu_flux2_dev", LoadSpec.from_dir(snap))
    d1 = dev.generate(GenerationRequest(**req)).images[0].pixels                         # embedded guidance 4
    d2 = dev.generate(GenerationRequest(**req, guidance=1.5)).images[0].pixels
    assert d1 != d2
    with pytest.raises(InferenceError):
        dev.generate(GenerationRequest(**req, negative_prompt="blurry"))
