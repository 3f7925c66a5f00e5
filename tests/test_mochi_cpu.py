"""Mochi 1: the dual-stream DiT against an independent restatement that keeps the padded text rows and masks them
(proving that passing valid rows only is the same computation), the causal decoder's chunked decode against the
one-shot decode and a direct 3-D convolution, the noise table, and provider conformance."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_mochi as M

CFG = M.MochiConfig(num_heads=2, head_dim=8, num_layers=3, pooled_dim=12, in_channels=4, text_embed_dim=16, time_embed_dim=8,
                    pool_heads=2)


def _direct(w, cfg, hidden, enc, mask, t):
    """hidden [C, F, H, W]; enc [L, E] padded; mask [L] 0/1."""
    C, Fr, H, W = hidden.shape
    p, nh, hd, D = cfg.patch_size, cfg.num_heads, cfg.head_dim, cfg.inner
    lin = lambda v, n: v @ w[n + ".weight"].t() + (w[n + ".bias"] if n + ".bias" in w else 0)      # noqa: E731
    rms = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + cfg.eps)                       # noqa: E731
    rmsw = lambda v, k: v / torch.sqrt((v * v).mean(-1, keepdim=True) + 1e-5) * w[k]               # noqa: E731
    half = cfg.time_embed_dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    te = lin(F.silu(lin(torch.cat([torch.cos(t * f), torch.sin(t * f)]), "time_embed.timestep_embedder.linear_1")),
             "time_embed.timestep_embedder.linear_2")
    # attention pool with masked keys
    L, E = enc.shape
    pool = (enc * (mask / mask.sum().clamp(min=1))[:, None]).sum(0, keepdim=True)
    kv = lin(torch.cat([pool, enc]), "time_embed.pooler.to_kv").view(L + 1, 2, cfg.pool_heads, -1)
    q = lin(pool, "time_embed.pooler.to_q").view(cfg.pool_heads, -1)
    s = torch.einsum("hd,khd->hk", q, kv[:, 0]) / math.sqrt(E // cfg.pool_heads)
    s[:, 1:] = s[:, 1:].masked_fill(mask[None] == 0, float("-inf"))
    temb = te + lin(torch.einsum("hk,khd->hd", s.softmax(-1), kv[:, 1]).reshape(E), "time_embed.pooler.to_out")
    txt = lin(enc, "time_embed.caption_proj")
    st = F.silu(temb)
    x = F.conv2d(hidden.permute(1, 0, 2, 3), w["patch_embed.proj.weight"], w["patch_embed.proj.bias"], stride=p)
    ph, pw = H // p, W // p
    hs = x.reshape(Fr, D, ph * pw).transpose(1, 2).reshape(Fr * ph * pw, D)
    ang = (M.mochi_positions(Fr, ph, pw) @ w["pos_frequencies"].reshape(3, -1)).reshape(-1, nh, hd // 2)

    def rot(v):
        vc = torch.view_as_complex(v.reshape(*v.shape[:-1], -1, 2).contiguous())
        return torch.view_as_real(vc * torch.polar(torch.ones_like(ang), ang)).flatten(-2)

    def glu(v, n):
        a, b = lin(v, n + ".net.0.proj").chunk(2, -1)
        return lin(a * F.silu(b), n + ".net.2")

    Sv = hs.shape[0]
    key_bias = torch.cat([torch.zeros(Sv), torch.where(mask > 0, 0.0, float("-inf"))])
    for i in range(cfg.num_layers):
        b, last = f"transformer_blocks.{i}", i == cfg.num_layers - 1
        a = b + ".attn1."
        sa, ga, sm, gm = lin(st, b + ".norm1.linear").chunk(4)
        n_h = rms(hs) * (1 + sa)
        if last:
            n_e = rms(txt) * (1 + lin(st, b + ".norm1_context.linear_1"))
        else:
            esa, ega, esm, egm = lin(st, b + ".norm1_context.linear").chunk(4)
            n_e = rms(txt) * (1 + esa)
        hv = lambda v: v.view(-1, nh, hd)       # noqa: E731
        q = torch.cat([rot(rmsw(hv(lin(n_h, a + "to_q")), a + "norm_q.weight")), rmsw(hv(lin(n_e, a + "add_q_proj")), a + "norm_added_q.weight")])
        k = torch.cat([rot(rmsw(hv(lin(n_h, a + "to_k")), a + "norm_k.weight")), rmsw(hv(lin(n_e, a + "add_k_proj")), a + "norm_added_k.weight")])
        v = torch.cat([hv(lin(n_h, a + "to_v")), hv(lin(n_e, a + "add_v_proj"))])
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd) + key_bias[None, None, :]
        o = torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(-1, D)
        hs = hs + rms(lin(o[:Sv], a + "to_out.0")) * torch.tanh(ga)
        hs = hs + rms(glu(rms(hs) * (1 + sm), b + ".ff")) * torch.tanh(gm)
        if not last:
            txt = txt + rms(lin(o[Sv:], a + "to_add_out")) * torch.tanh(ega)
            txt = txt + rms(glu(rms(txt) * (1 + esm), b + ".ff_context")) * torch.tanh(egm)
    scale, shift = lin(st, "norm_out.linear").chunk(2)
    out = lin(F.layer_norm(hs, (D,), eps=1e-6) * (1 + scale) + shift, "proj_out")
    return out.reshape(Fr, ph, pw, p, p, C).permute(5, 0, 1, 3, 2, 4).reshape(C, Fr, H, W)


def test_dit_matches_masked_restatement():
    torch.manual_seed(0)
    w = M.random_mochi_weights(CFG, seed=4, std=0.2)
    model = M.MochiDiT(CFG, w)
    hidden = torch.randn(1, 4, 2, 4, 6)
    L, n = 7, 4
    enc = torch.randn(1, L, 16)
    mask = torch.tensor([1.0] * n + [0.0] * (L - n))
    t = torch.tensor([412.0])
    got = model.forward(hidden, enc[:, :n], t)
    want = _direct(w, CFG, hidden[0], enc[0], mask, t[0])
    assert got.shape == hidden.shape and torch.allclose(got[0], want, atol=3e-4, rtol=1e-3), (got[0] - want).abs().max()


def test_positions_and_noise_table():
    pos = M.mochi_positions(2, 4, 4)
    assert pos.shape == (32, 3) and pos[0].tolist() == [0.0, -72.0, -72.0] and pos[17].tolist() == [1.0, -72.0, -24.0]
    s = M.linear_quadratic_sigmas(64)
    assert len(s) == 64 and s[0] == 1.0 and all(a > b for a, b in zip(s, s[1:])) and s[-1] > 0.0
    assert abs(s[32] - (1.0 - 0.025)) < 1e-9 and abs((s[0] - s[1]) - 0.025 / 32) < 1e-12       # linear half removes 0.025
    full = M.MochiConfig()
    assert full.inner == 3072 and full.ff_inner == 8192 and full.ff_ctx_inner == 4096


def test_decoder_chunked_equals_one_shot_and_direct_conv():
    cfg = M.MochiVaeConfig(decoder_block_out_channels=(8, 8, 8, 16), layers_per_block=(1, 1, 1, 1, 1), groups=4,
                           latents_mean=tuple([0.1] * 12), latents_std=tuple([1.5] * 12))
    dec = M.MochiVaeDecoder(cfg, M.random_mochi_vae_weights(cfg, seed=2))
    z = torch.randn(1, 12, 3, 2, 3)
    full = dec.decode(z)
    assert full.shape == (1, 3, (3 - 1) * 6 + 1, 16, 24)
    for chunk in (1, 2):
        assert torch.allclose(dec.decode(z, chunk), full, atol=1e-5)
    # one causal convolution against the textbook form: pad 2 copies of the first frame, replicate-pad space
    x = torch.randn(1, 16, 3, 4, 5)
    name = "block_in.resnets.0.conv1.conv"
    got = dec._conv(x, name, None)
    xp = F.pad(torch.cat([x[:, :, :1]] * 2 + [x], 2), (1, 1, 1, 1, 0, 0), mode="replicate")
    assert torch.allclose(got, F.conv3d(xp, dec.w[name + ".weight"], dec.w[name + ".bias"]), atol=1e-5)


def test_mochi_provider_conforms(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.mochi import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "mochi")
    reg = provider_registry("cpu")
    assert "cpu_mochi_1" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_mochi_1", LoadSpec.from_dir(snap))
    kit.conformance(gen, kit.Profile(width=64, height=64, steps=2, cancel_steps=4))
    out = gen.generate(GenerationRequest(prompt="a paper boat", width=64, height=64, steps=2, seed=1, frames=7))
    assert len(out.video_frames) == 7 and out.fps == 30 and len(out.video_frames[0].pixels) == 64 * 64 * 3
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(prompt="x", width=64, height=64, steps=2, frames=8))
