"""Chroma DiT: the converted-checkpoint oracle against an independent restatement in the checkpoint's own layout
(separate q / k / v projections, modulation rows read straight from the Approximator table)."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_chroma as C
from inference_b200.models.dit_flux import make_ids, rope_table

CFG = C.ChromaConfig(in_channels=16, num_layers=2, num_single_layers=3, attention_head_dim=16, num_attention_heads=2,
                     joint_attention_dim=24, axes_dims_rope=(4, 6, 6), approximator_num_channels=16,
                     approximator_hidden_dim=40, approximator_layers=2)


def _direct(w, cfg, img, txt, t, cos, sin):
    H, nh, hd = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda x, n: F.linear(x, w[n + ".weight"], w[n + ".bias"])
    ln = lambda x: F.layer_norm(x, (H,), eps=1e-6)
    rms = lambda x, s: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * s
    mod = lambda x, sc, sh: ln(x) * (1 + sc) + sh

    def rope(x):                                    # [B, S, heads, hd], interleaved pairs
        x0, x1 = x[..., 0::2], x[..., 1::2]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), -1).flatten(-2)

    def heads(x, norm=None):
        x = x.view(x.shape[0], x.shape[1], nh, hd)
        return rms(x, w[norm]) if norm else x

    def attend(q, k, v):
        o = F.scaled_dot_product_attention(rope(q).transpose(1, 2), rope(k).transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).flatten(-2)
    # approximator
    nc = cfg.approximator_num_channels // 4
    emb = lambda v, d: torch.cat([(v[:, None] * torch.exp(torch.arange(d // 2) * (-math.log(10000.0) / (d // 2)))).cos(),
                                  (v[:, None] * torch.exp(torch.arange(d // 2) * (-math.log(10000.0) / (d // 2)))).sin()], -1)
    n = cfg.mod_index_len
    x = torch.cat([emb(t * 1000, nc), emb(torch.zeros_like(t), nc)], -1)[:, None].expand(-1, n, -1)
    x = torch.cat([x, emb(torch.arange(n).float() * 1000, 2 * nc)[None].expand(t.numel(), -1, -1)], -1)
    a = "distilled_guidance_layer."
    x = lin(x, a + "in_proj")
    for i in range(cfg.approximator_layers):
        nx = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + C.APPROX_RMS_EPS) * w[f"{a}norms.{i}.weight"]
        x = x + lin(F.silu(lin(nx, f"{a}layers.{i}.linear_1")), f"{a}layers.{i}.linear_2")
    tab = lin(x, a + "out_proj")
    row = lambda j: tab[:, j:j + 1]
    h, e = lin(img, "x_embedder"), lin(txt, "context_embedder")
    St = e.shape[1]
    ns, nd = cfg.num_single_layers, cfg.num_layers
    for i in range(nd):
        p = f"transformer_blocks.{i}"
        io, to = 3 * ns + 6 * i, 3 * ns + 6 * nd + 6 * i
        nh_, ne = mod(h, row(io + 1), row(io)), mod(e, row(to + 1), row(to))
        q = torch.cat([heads(lin(ne, p + ".attn.add_q_proj"), p + ".attn.norm_added_q.weight"),
                       heads(lin(nh_, p + ".attn.to_q"), p + ".attn.norm_q.weight")], 1)
        k = torch.cat([heads(lin(ne, p + ".attn.add_k_proj"), p + ".attn.norm_added_k.weight"),
                       heads(lin(nh_, p + ".attn.to_k"), p + ".attn.norm_k.weight")], 1)
        v = torch.cat([heads(lin(ne, p + ".attn.add_v_proj")), heads(lin(nh_, p + ".attn.to_v"))], 1)
        o = attend(q, k, v)
        h = h + row(io + 2) * lin(o[:, St:], p + ".attn.to_out.0")
        ff = lambda z, pre: lin(F.gelu(lin(z, pre + ".net.0.proj"), approximate="tanh"), pre + ".net.2")
        h = h + row(io + 5) * ff(mod(h, row(io + 4), row(io + 3)), p + ".ff")
        e = e + row(to + 2) * lin(o[:, :St], p + ".attn.to_add_out")
        e = e + row(to + 5) * ff(mod(e, row(to + 4), row(to + 3)), p + ".ff_context")
    j = torch.cat([e, h], 1)
    for i in range(ns):
        p = f"single_transformer_blocks.{i}"
        nj = mod(j, row(3 * i + 1), row(3 * i))
        o = attend(heads(lin(nj, p + ".attn.to_q"), p + ".attn.norm_q.weight"),
                   heads(lin(nj, p + ".attn.to_k"), p + ".attn.norm_k.weight"), heads(lin(nj, p + ".attn.to_v")))
        j = j + row(3 * i + 2) * lin(torch.cat([o, F.gelu(lin(nj, p + ".proj_mlp"), approximate="tanh")], -1), p + ".proj_out")
    return lin(mod(j[:, St:], row(n - 1), row(n - 2)), "proj_out")


def test_chroma_oracle_matches_direct_restatement():
    assert CFG.mod_index_len == 3 * 3 + 12 * 2 + 2 and C.ChromaConfig().mod_index_len == 344
    w = C.random_chroma_weights(CFG, seed=1, std=0.08)
    g = torch.Generator().manual_seed(0)
    img, txt = torch.randn(1, 12, 16, generator=g), torch.randn(1, 5, 24, generator=g)
    t = torch.tensor([0.7])
    txt_ids, img_ids = make_ids(3, 4, 5)
    cos, sin = rope_table(torch.cat([txt_ids, img_ids], 0), CFG.axes_dims_rope, 10000.0)
    model = C.OracleChromaDiT(CFG, w)
    got = model.forward(img, img_ids, txt, txt_ids, t, None)
    want = _direct(w, CFG, img, txt, t, cos, sin)
    assert got.shape == (1, 12, 16)
    torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-4)
    other = model.forward(img, img_ids, txt, txt_ids, torch.tensor([0.2]), None)
    assert float((other - got).abs().max()) > 1e-4               # the timestep reaches every modulation
    x = C.approximator_input(torch.tensor([0.0]), CFG)
    assert x.shape == (1, CFG.mod_index_len, 16) and torch.allclose(x[0, 0, :2], torch.ones(2))    # cos block first
    conv = C.convert_chroma_weights(w, CFG)
    assert conv["single_blocks.0.linear1.weight"].shape == (3 * 32 + 4 * 32, 32)
    assert conv["double_blocks.1.txt_attn.qkv.bias"].shape == (96,)


# ---- providers ---------------------------------------------------------------------------------------------------------------
def test_sigma_schedules():
    import scipy.stats

    from inference_b200.media.chroma import ChromaVariant, beta_ppf, chroma_sigmas

    for p in (0.01, 0.2, 0.5, 0.77, 0.999):
        assert abs(beta_ppf(p) - scipy.stats.beta.ppf(p, 0.6, 0.6)) < 1e-9
    hd = chroma_sigmas(ChromaVariant.HD, 28)
    assert len(hd) == 29 and hd[0] == 1.0 and hd[-1] == 0.0
    raw = 1.0 / 28
    assert abs(hd[-2] - 3.0 * raw / (1 + 2.0 * raw)) < 1e-12
    assert all(a > b for a, b in zip(hd, hd[1:]))
    base = chroma_sigmas(ChromaVariant.BASE, 28)
    assert abs(base[0] - 1.0) < 1e-12 and abs(base[-2] - raw) < 1e-12 and all(a > b for a, b in zip(base, base[1:]))
    flash = chroma_sigmas(ChromaVariant.FLASH, 8)
    assert flash == [1.0 + (1 / 8 - 1.0) * i / 7 for i in range(8)] + [0.0]


def test_vae_key_conversion_round_trips():
    from inference_b200.media.chroma import convert_diffusers_vae_decoder, native_vae_to_diffusers
    from inference_b200.models.vae import VaeConfig, random_vae_weights

    native = random_vae_weights(VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1), 3)
    native = {k: v for k, v in native.items() if k.startswith("decoder.")}
    dif = native_vae_to_diffusers(native)
    assert "decoder.mid_block.attentions.0.to_q.weight" in dif and dif["decoder.mid_block.attentions.0.to_q.weight"].dim() == 2
    assert "decoder.up_blocks.0.resnets.0.conv1.weight" in dif and "decoder.conv_norm_out.weight" in dif
    back = convert_diffusers_vae_decoder(dif)
    assert back.keys() == native.keys()
    assert all(torch.equal(back[k], native[k]) for k in native)


def test_chroma_providers_conform(tmp_path):
    from inference_b200.contracts.errors import Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec, Quant, WeightsSource
    from inference_b200.media import provider_registry
    from inference_b200.media.chroma import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit
    import pytest

    snap = write_synthetic_snapshot(tmp_path / "chroma")
    reg = provider_registry("cpu")
    assert [i for i in reg.ids() if "chroma" in i] == ["cpu_chroma1_hd", "cpu_chroma1_base", "cpu_chroma1_flash"]
    assert reg.descriptor_conformance_errors() == []
    g = reg.load("cpu_chroma1_flash", LoadSpec.from_dir(snap))
    kit.conformance(g, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_chroma1_flash", LoadSpec.from_dir(snap))
    with pytest.raises(Unsupported):
        reg.load("cpu_chroma1_hd", LoadSpec(weights=WeightsSource.dir(snap), quantize=Quant.Q4))
    # true CFG: two forwards per step; guidance 1 and the negative prompt's absence take the single-forward path
    hd = reg.load("cpu_chroma1_hd", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    a = hd.generate(GenerationRequest(**req, true_cfg=1.0)).images[0].pixels
    b = hd.generate(GenerationRequest(**req, true_cfg=3.0, negative_prompt="blurry")).images[0].pixels
    c = hd.generate(GenerationRequest(**req, true_cfg=3.0, negative_prompt="blurry")).images[0].pixels
    assert b == c and a != b and len(a) == 256 * 256 * 3
