"""Qwen-Image: the converted-checkpoint oracle against a restatement in the checkpoint's own layout, the single-frame
autoencoder against causal 3-D convolutions, position ids, schedule and guidance helpers, provider conformance."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.models import dit_qwen_image as Q
from inference_b200.models.dit_flux import rope_table

CFG = Q.QwenImageConfig(in_channels=16, num_layers=2, attention_head_dim=16, num_attention_heads=2, joint_attention_dim=24,
                        axes_dims_rope=(4, 6, 6))


def _direct(w, cfg, img, txt, t, cos, sin):
    H, nh, hd = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda x, n: F.linear(x, w[n + ".weight"], w[n + ".bias"])                  # noqa: E731
    ln = lambda x: F.layer_norm(x, (H,), eps=1e-6)                                    # noqa: E731
    rms = lambda x, s: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * s    # noqa: E731

    def rope(x):
        xc = torch.view_as_complex(x.double().reshape(*x.shape[:-1], -1, 2))
        fr = torch.complex(cos.double(), sin.double())[None, :, None, :]
        return torch.view_as_real(xc * fr).flatten(-2).float()

    def heads(x, norm=None):
        x = x.view(x.shape[0], x.shape[1], nh, hd)
        return rms(x, w[norm]) if norm else x

    half = 128
    fr = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half) * (t * 1000.0)
    temb = lin(F.silu(lin(torch.cat([fr.cos(), fr.sin()])[None], "time_text_embed.timestep_embedder.linear_1")),
               "time_text_embed.timestep_embedder.linear_2")
    sv = F.silu(temb)
    h = lin(img, "img_in")
    e = lin(rms(txt, w["txt_norm.weight"]), "txt_in")
    St = e.shape[1]
    ff = lambda z, pre: lin(F.gelu(lin(z, pre + ".net.0.proj"), approximate="tanh"), pre + ".net.2")   # noqa: E731
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        im1, im2 = lin(sv, p + ".img_mod.1")[:, None].chunk(2, -1)
        tm1, tm2 = lin(sv, p + ".txt_mod.1")[:, None].chunk(2, -1)
        (ish, isc, ig), (tsh, tsc, tg) = im1.chunk(3, -1), tm1.chunk(3, -1)
        nh_, ne = ln(h) * (1 + isc) + ish, ln(e) * (1 + tsc) + tsh
        q = torch.cat([heads(lin(ne, p + ".attn.add_q_proj"), p + ".attn.norm_added_q.weight"),
                       heads(lin(nh_, p + ".attn.to_q"), p + ".attn.norm_q.weight")], 1)
        k = torch.cat([heads(lin(ne, p + ".attn.add_k_proj"), p + ".attn.norm_added_k.weight"),
                       heads(lin(nh_, p + ".attn.to_k"), p + ".attn.norm_k.weight")], 1)
        v = torch.cat([heads(lin(ne, p + ".attn.add_v_proj")), heads(lin(nh_, p + ".attn.to_v"))], 1)
        o = F.scaled_dot_product_attention(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2))
        o = o.transpose(1, 2).flatten(-2)
        h = h + ig * lin(o[:, St:], p + ".attn.to_out.0")
        e = e + tg * lin(o[:, :St], p + ".attn.to_add_out")
        (ish, isc, ig), (tsh, tsc, tg) = im2.chunk(3, -1), tm2.chunk(3, -1)
        h = h + ig * ff(ln(h) * (1 + isc) + ish, p + ".img_mlp")
        e = e + tg * ff(ln(e) * (1 + tsc) + tsh, p + ".txt_mlp")
    scale, shift = lin(sv, "norm_out.linear")[:, None].chunk(2, -1)
    return lin(ln(h) * (1 + scale) + shift, "proj_out")


def test_oracle_matches_direct_restatement():
    w = Q.random_qwen_image_weights(CFG, seed=1, std=0.08)
    g = torch.Generator().manual_seed(0)
    img, txt = torch.randn(1, 12, 16, generator=g), torch.randn(1, 5, 24, generator=g)
    t = torch.tensor([0.7])
    txt_ids, img_ids = Q.position_ids(3, 4, 5)
    cos, sin = rope_table(torch.cat([txt_ids, img_ids], 0), CFG.axes_dims_rope, 10000.0)
    model = Q.OracleQwenImageDiT(CFG, w)
    got = model.forward(img, img_ids, model.prepare_text(txt), txt_ids, t, None)
    want = _direct(w, CFG, img, txt, t[0], cos, sin)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-4)


def test_position_ids():
    txt, img = Q.position_ids(5, 4, 3)
    assert img[:, 0].abs().sum() == 0
    assert img.view(5, 4, 3)[:, 0, 1].tolist() == [-3.0, -2.0, -1.0, 0.0, 1.0]          # rows centred: r - (5 - 5 // 2)
    assert img.view(5, 4, 3)[0, :, 2].tolist() == [-2.0, -1.0, 0.0, 1.0]
    assert txt.tolist() == [[2.0] * 3, [3.0] * 3, [4.0] * 3]                             # from max(5 // 2, 4 // 2)


def test_single_frame_autoencoder_equals_causal_3d_convolutions():
    from inference_b200.models.vae_qwen import LATENTS_MEAN, LATENTS_STD, QwenVaeConfig, QwenVaeDecoder, random_qwen_vae_weights

    cfg = QwenVaeConfig(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    w = random_qwen_vae_weights(cfg, seed=3, std=0.2)
    z = torch.randn(1, 16, 3, 5, generator=torch.Generator().manual_seed(1))
    out = QwenVaeDecoder(cfg, w).decode(z)
    assert out.shape == (1, 3, 24, 40)

    def cconv(x, name, pad):                 # causal in time: two zero frames in front for a 3-tap kernel
        k = w[name + ".weight"].shape[2]
        x = F.pad(x, (pad, pad, pad, pad, k - 1, 0))
        return F.conv3d(x, w[name + ".weight"], w[name + ".bias"])

    def norm(x, name):
        g = w[name + ".gamma"].reshape(1, -1, 1, 1, 1)
        return x / torch.sqrt(x.pow(2).sum(1, keepdim=True) + 1e-12) * x.shape[1] ** 0.5 * g

    def res(x, p):
        h = cconv(F.silu(norm(x, p + ".norm1")), p + ".conv1", 1)
        h = cconv(F.silu(norm(h, p + ".norm2")), p + ".conv2", 1)
        return h + (cconv(x, p + ".conv_shortcut", 0) if p + ".conv_shortcut.weight" in w else x)

    x = z * torch.tensor(LATENTS_STD).view(1, -1, 1, 1) + torch.tensor(LATENTS_MEAN).view(1, -1, 1, 1)
    h = cconv(cconv(x[:, :, None], "post_quant_conv", 0), "decoder.conv_in", 1)
    h = res(h, "decoder.mid_block.resnets.0")
    a = "decoder.mid_block.attentions.0"
    f2 = h[:, :, 0]
    qkv = F.conv2d(norm(h, a + ".norm")[:, :, 0], w[a + ".to_qkv.weight"], w[a + ".to_qkv.bias"])
    C = f2.shape[1]
    q, k, v = qkv.reshape(1, 3, C, -1).unbind(1)
    att = torch.softmax(q.transpose(1, 2) @ k / C ** 0.5, -1) @ v.transpose(1, 2)
    h = (f2 + F.conv2d(att.transpose(1, 2).reshape(f2.shape), w[a + ".proj.weight"], w[a + ".proj.bias"]))[:, :, None]
    h = res(h, "decoder.mid_block.resnets.1")
    for i, (_, _, up) in enumerate(cfg.up_plan()):
        for j in range(cfg.num_res_blocks + 1):
            h = res(h, f"decoder.up_blocks.{i}.resnets.{j}")
        if up is not None:
            u = f"decoder.up_blocks.{i}.upsamplers.0.resample.1"
            h = F.conv2d(F.interpolate(h[:, :, 0], scale_factor=2, mode="nearest"), w[u + ".weight"], w[u + ".bias"],
                         padding=1)[:, :, None]
    ref = cconv(F.silu(norm(h, "decoder.norm_out")), "decoder.conv_out", 1)[:, :, 0]
    torch.testing.assert_close(out, ref, atol=1e-4, rtol=1e-4)


def test_schedule_and_guidance_helpers():
    from inference_b200.media.qwen_image import guided_velocity, qwen_mu, qwen_sigmas

    assert abs(qwen_mu(256, 256) - 0.5) < 1e-9 and abs(qwen_mu(1024, 1024) - (0.5 + 0.4 * (4096 - 256) / (8192 - 256))) < 1e-9
    s = qwen_sigmas(20, 1024, 1024)
    assert len(s) == 21 and s[0] == 1.0 and s[-1] == 0.0 and abs(s[19] - 0.02) < 1e-9
    assert all(a > b for a, b in zip(s, s[1:]))
    g = torch.Generator().manual_seed(0)
    pos, neg = torch.randn(1, 5, 8, generator=g), torch.randn(1, 5, 8, generator=g)
    v = guided_velocity(pos, neg, 4.0)
    torch.testing.assert_close(v.norm(dim=-1), pos.norm(dim=-1))
    comb = neg + 4.0 * (pos - neg)
    torch.testing.assert_close(v / v.norm(dim=-1, keepdim=True), comb / comb.norm(dim=-1, keepdim=True))


def test_qwen_image_provider_conforms(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.qwen_image import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "qi", text="qwen_vl")
    reg = provider_registry("cpu")
    assert "cpu_qwen_image" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_qwen_image", LoadSpec.from_dir(snap))
    kit.conformance(gen, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_qwen_image", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = gen.generate(GenerationRequest(**req, true_cfg=1.0)).images[0].pixels
    b = gen.generate(GenerationRequest(**req)).images[0].pixels                     # default true CFG 4, negative " "
    c = gen.generate(GenerationRequest(**req, guidance=4.0, negative_prompt=" ")).images[0].pixels
    assert b == c and a != b and len(a) == 256 * 256 * 3
