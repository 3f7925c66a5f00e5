"""Anima: the Cosmos DiT and the text conditioner against independent restatements, rotary / sigma / key-conversion
values stated by the reference's tests, adapter folding with strict routing, and provider conformance."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.models import dit_anima as A

CFG = A.CosmosConfig(num_attention_heads=2, attention_head_dim=12, num_layers=2, text_embed_dim=10, adaln_lora_dim=6,
                     in_channels=4, out_channels=4, max_size=(4, 16, 16))
CCFG = A.ConditionerConfig(source_dim=14, target_dim=10, model_dim=8, num_layers=2, num_attention_heads=2,
                           target_vocab_size=50, min_sequence_length=9)


def _rot_half(x, ang):                      # x [S, nh, hd]; ang [S, hd/2]; rotate_half convention
    c, s = torch.cat([ang.cos(), ang.cos()], -1)[:, None], torch.cat([ang.sin(), ang.sin()], -1)[:, None]
    h = x.shape[-1] // 2
    return x * c + torch.cat([-x[..., h:], x[..., :h]], -1) * s


def _mha(q, k, v):
    s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(q.shape[-1])
    return torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(q.shape[0], -1)


def _direct_dit(w, cfg, lat, sigma, enc):
    C, T, Hl, Wl = lat.shape
    H, nh, hd = cfg.hidden, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda v, n: v @ w[n + ".weight"].t()                       # noqa: E731
    ln = lambda v: F.layer_norm(v, (H,), eps=1e-6)                    # noqa: E731
    rms = lambda v, k, e: v / torch.sqrt((v * v).mean(-1, keepdim=True) + e) * w[k]      # noqa: E731
    x = torch.cat([lat, torch.zeros(1, T, Hl, Wl)], 0)
    toks, ang = [], []
    dh = hd // 6 * 2
    dt = hd - 2 * dh
    fr = lambda sc, d: torch.tensor([1.0 / (10000.0 * sc ** (d / (d - 2.0))) ** (2.0 * k / d) for k in range(d // 2)], dtype=torch.float64)  # noqa: E731
    for t in range(T):
        for i in range(Hl // 2):
            for j in range(Wl // 2):
                toks.append(x[:, t:t + 1, 2 * i:2 * i + 2, 2 * j:2 * j + 2].reshape(-1))
                ang.append(torch.cat([t * fr(cfg.rope_scale[0], dt), i * fr(cfg.rope_scale[1], dh), j * fr(cfg.rope_scale[2], dh)]))
    h = lin(torch.stack(toks), "x_embedder.proj.1")
    ang = torch.stack(ang).float()
    half = H // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    proj = torch.cat([torch.cos(sigma * f), torch.sin(sigma * f)])
    temb = lin(F.silu(lin(proj, "t_embedder.1.linear_1")), "t_embedder.1.linear_2")
    emb = F.silu(rms(proj, "t_embedding_norm.weight", 1e-6))

    def attn(xn, src, p, rope):
        q = rms(lin(xn, p + ".q_proj").view(-1, nh, hd), p + ".q_norm.weight", 1e-5)
        k = rms(lin(src, p + ".k_proj").view(-1, nh, hd), p + ".k_norm.weight", 1e-5)
        v = lin(src, p + ".v_proj").view(-1, nh, hd)
        if rope:
            q, k = _rot_half(q, ang), _rot_half(k, ang)
        return lin(_mha(q, k, v), p + ".output_proj")

    for i in range(cfg.num_layers):
        b = f"blocks.{i}"
        for name, fn in (("self_attn", lambda xn: attn(xn, xn, b + ".self_attn", True)),
                         ("cross_attn", lambda xn: attn(xn, enc, b + ".cross_attn", False)),
                         ("mlp", lambda xn: lin(F.gelu(lin(xn, b + ".mlp.layer1")), b + ".mlp.layer2"))):
            sh, sc, g = (lin(lin(emb, f"{b}.adaln_modulation_{name}.1"), f"{b}.adaln_modulation_{name}.2") + temb).chunk(3)
            h = h + g * fn(ln(h) * (1 + sc) + sh)
    sh, sc = (lin(lin(emb, "final_layer.adaln_modulation.1"), "final_layer.adaln_modulation.2") + temb[: 2 * H]).chunk(2)
    out = lin(ln(h) * (1 + sc) + sh, "final_layer.linear")            # [S, ph * pw * pt * oc]
    res = torch.zeros(cfg.out_channels, T, Hl, Wl)
    n = 0
    for t in range(T):
        for i in range(Hl // 2):
            for j in range(Wl // 2):
                res[:, t, 2 * i:2 * i + 2, 2 * j:2 * j + 2] = out[n].view(2, 2, 1, cfg.out_channels).permute(3, 2, 0, 1)[:, 0]
                n += 1
    return res


def _direct_conditioner(w, cfg, src, ids):
    hd, nh = cfg.head_dim, cfg.num_attention_heads
    pre = "llm_adapter."
    lin = lambda v, n: v @ w[pre + n + ".weight"].t() + (w[pre + n + ".bias"] if pre + n + ".bias" in w else 0)      # noqa: E731
    rms = lambda v, k: v / torch.sqrt((v * v).mean(-1, keepdim=True) + cfg.norm_eps) * w[pre + k]                    # noqa: E731
    ang = lambda n: torch.arange(n).float()[:, None] * torch.tensor([cfg.rope_theta ** (-2.0 * i / hd) for i in range(hd // 2)])[None]      # noqa: E731
    h = w[pre + "embed.weight"][ids]
    ta, sa = ang(len(ids)), ang(src.shape[0])

    def attn(xn, kv, p, ka):
        q = _rot_half(rms(lin(xn, p + ".q_proj").view(-1, nh, hd), p + ".q_norm.weight"), ta)
        k = _rot_half(rms(lin(kv, p + ".k_proj").view(-1, nh, hd), p + ".k_norm.weight"), ka)
        return lin(_mha(q, k, lin(kv, p + ".v_proj").view(-1, nh, hd)), p + ".o_proj")

    for i in range(cfg.num_layers):
        b = f"blocks.{i}"
        n = rms(h, b + ".norm_self_attn.weight")
        h = h + attn(n, n, b + ".self_attn", ta)
        h = h + attn(rms(h, b + ".norm_cross_attn.weight"), src, b + ".cross_attn", sa)
        h = h + lin(F.gelu(lin(rms(h, b + ".norm_mlp.weight"), b + ".mlp.0")), b + ".mlp.2")
    h = rms(lin(h, "out_proj"), "norm.weight")
    return torch.cat([h, torch.zeros(cfg.min_sequence_length - len(ids), h.shape[1])])


def test_dit_and_conditioner_match_restatements():
    torch.manual_seed(0)
    w = A.random_anima_weights(CFG, CCFG, seed=5, std=0.2)
    lat, enc = torch.randn(1, 4, 2, 4, 6), torch.randn(1, 7, 10)
    sigma = torch.tensor([0.63])
    got = A.CosmosDiT(CFG, w).forward(lat, sigma, enc)
    want = _direct_dit(w, CFG, lat[0], sigma[0], enc[0])
    assert got.shape == lat.shape and torch.allclose(got[0], want, atol=3e-4, rtol=1e-3), (got[0] - want).abs().max()
    src, ids = torch.randn(1, 5, 14), torch.tensor([[3, 17, 42, 9]])
    c = A.AnimaTextConditioner(CCFG, w).forward(src, ids)
    want_c = _direct_conditioner(w, CCFG, src[0], ids[0])
    assert c.shape == (1, 9, 10) and torch.allclose(c[0], want_c, atol=2e-4, rtol=1e-3), (c[0] - want_c).abs().max()
    assert torch.equal(c[0, 4:], torch.zeros(5, 10))


def test_sigmas_prefix_and_vae_keys_match_reference_values():
    s = A.anima_sigmas(10)
    assert len(s) == 11 and abs(s[0] - 1.0) < 1e-6 and abs(s[1] - 2.7 / 2.8) < 1e-5 and abs(s[9] - 0.25) < 1e-5 and s[10] == 0.0
    assert A.anima_sigmas(1) == [1.0, 0.0] and len(A.anima_sigmas(30)) == 31
    for root in ("net", "model.diffusion_model"):
        keys = [f"{root}.llm_adapter.embed.weight", f"{root}.x_embedder.proj.1.weight", f"{root}.blocks.0.mlp.layer1.weight"]
        assert A.detect_dit_prefix(keys) == root
    with pytest.raises(ValueError):
        A.detect_dit_prefix(["foo.weight"])
    cv = A.convert_vae_key
    assert cv("conv1.weight") == "quant_conv.weight" and cv("conv2.bias") == "post_quant_conv.bias"
    assert cv("encoder.conv1.weight") == "encoder.conv_in.weight" and cv("decoder.conv1.bias") == "decoder.conv_in.bias"
    assert cv("encoder.head.0.gamma") == "encoder.norm_out.gamma" and cv("decoder.head.2.weight") == "decoder.conv_out.weight"
    assert cv("encoder.downsamples.0.residual.2.weight") == "encoder.down_blocks.0.conv1.weight"
    assert cv("decoder.upsamples.3.resample.1.weight") == "decoder.up_blocks.0.upsamplers.0.resample.1.weight"
    assert cv("decoder.upsamples.5.residual.6.bias") == "decoder.up_blocks.1.resnets.1.conv2.bias"
    assert cv("decoder.middle.1.to_qkv.weight") == "decoder.mid_block.attentions.0.to_qkv.weight"
    assert cv("decoder.middle.2.residual.0.gamma") == "decoder.mid_block.resnets.1.norm1.gamma"
    cos, sin = A.cosmos_rope(A.CosmosConfig(), 1, 2, 3)
    assert cos.shape == (6, 64) and torch.allclose(cos[0], torch.ones(64)) and torch.allclose(cos[:, :22], torch.ones(6, 22))
    assert abs(cos[1, 43].item() - math.cos(1.0)) < 1e-6 and abs(sin[3, 22].item() - math.sin(1.0)) < 1e-6
    with pytest.raises(ValueError):
        A.cosmos_rope(A.CosmosConfig(), 1, 121, 3)


def test_anima_providers_conform_and_fold_adapters(tmp_path):
    from inference_b200.contracts.errors import LoadError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.runtime import AdapterKind, AdapterSpec
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media import provider_registry
    from inference_b200.media.anima import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "anima", prefix="model.diffusion_model")
    reg = provider_registry("cpu")
    assert sorted(i for i in reg.ids() if "anima" in i) == ["cpu_anima_aesthetic", "cpu_anima_base", "cpu_anima_turbo"]
    assert reg.descriptor_conformance_errors() == []
    base = reg.load("cpu_anima_base", LoadSpec.from_dir(snap))
    d = base.descriptor().capabilities
    assert d.supports_lora and d.supports_lokr and d.supports_negative_prompt and d.min_size == 512 and d.max_size == 1536
    kit.conformance(base, kit.Profile(width=512, height=512, steps=2, cancel_steps=4))
    turbo = reg.load("cpu_anima_turbo", LoadSpec.from_dir(snap))
    assert not turbo.descriptor().capabilities.supports_negative_prompt
    kit.conformance(turbo, kit.Profile(width=512, height=512, steps=2, cancel_steps=4))
    req = GenerationRequest(prompt="a heron", width=512, height=512, steps=2, seed=3)
    plain = base.generate(req).images[0].pixels
    g = torch.Generator().manual_seed(1)
    lora = tmp_path / "l.safetensors"
    save_file({"diffusion_model.blocks.0.self_attn.q_proj.lora_A.weight": torch.randn(2, 24, generator=g),
               "diffusion_model.blocks.0.self_attn.q_proj.lora_B.weight": torch.randn(24, 2, generator=g),
               "lora_unet_llm_adapter_blocks_1_mlp_0.lora_down.weight": torch.randn(2, 16, generator=g),
               "lora_unet_llm_adapter_blocks_1_mlp_0.lora_up.weight": torch.randn(64, 2, generator=g),
               "lora_unet_llm_adapter_blocks_1_mlp_0.alpha": torch.tensor(1.0)}, lora)
    lokr = tmp_path / "k.safetensors"
    save_file({"lycoris_blocks_1_mlp_layer2.lokr_w1": torch.randn(4, 8, generator=g),
               "lycoris_blocks_1_mlp_layer2.lokr_w2": torch.randn(6, 12, generator=g) * 0.3}, lokr)
    spec = LoadSpec.from_dir(snap)
    spec.adapters = [AdapterSpec(path=str(lora), scale=1.0, kind=AdapterKind.LORA), AdapterSpec(path=str(lokr), scale=0.5, kind=AdapterKind.LOKR)]
    adapted = reg.load("cpu_anima_base", spec)
    assert adapted.generate(req).images[0].pixels != plain
    bad = tmp_path / "bad.safetensors"
    save_file({"blocks.9.nope.lora_A.weight": torch.zeros(1, 4), "blocks.9.nope.lora_B.weight": torch.zeros(4, 1)}, bad)
    spec.adapters = [AdapterSpec(path=str(bad), scale=1.0, kind=AdapterKind.LORA)]
    with pytest.raises(LoadError):
        reg.load("cpu_anima_base", spec).generate(req)
