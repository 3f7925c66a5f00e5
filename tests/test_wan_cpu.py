"""Wan video DiT against an independent restatement (3-D patch convolution, complex rotary, einsum attention), the
video autoencoder's invariants, the two-expert schedule and provider conformance."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.models import dit_wan as W

CFG = W.WanConfig(num_attention_heads=2, attention_head_dim=12, num_layers=2, ffn_dim=40, in_channels=4, out_channels=4,
                  text_dim=10, freq_dim=16)


def _direct(w, cfg, z, t, ctx):
    D, nh, hd = cfg.dim, cfg.num_attention_heads, cfg.attention_head_dim
    lin = lambda x, n: x @ w[n + ".weight"].t() + w[n + ".bias"]                     # noqa: E731
    ln = lambda x: F.layer_norm(x, (D,), eps=1e-6)                                    # noqa: E731
    rms = lambda x, n: x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w[n + ".weight"]   # noqa: E731
    C, Fr, H, Wd = z.shape
    x = F.conv3d(z[None], w["patch_embedding.weight"], w["patch_embedding.bias"], stride=(1, 2, 2))[0]     # [D, F, h, w]
    f, h, ww = x.shape[1:]
    x = x.flatten(1).t()
    axes = cfg.rope_axes
    fr = []
    for pos, d in zip(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(ww), indexing="ij"), axes):
        inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).double() / d))
        fr.append(torch.polar(torch.ones(f * h * ww, d // 2, dtype=torch.float64), pos.reshape(-1, 1).double() * inv))
    fr = torch.cat(fr, -1)

    def rope(u):
        uc = torch.view_as_complex(u.double().reshape(u.shape[0], nh, hd // 2, 2))
        return torch.view_as_real(uc * fr[:, None]).flatten(-2).float()

    def attn(xq, xkv, p, rot):
        q = rms(lin(xq, p + ".to_q"), p + ".norm_q").view(-1, nh, hd)
        k = rms(lin(xkv, p + ".to_k"), p + ".norm_k").view(-1, nh, hd)
        v = lin(xkv, p + ".to_v").view(-1, nh, hd)
        if rot:
            q, k = rope(q), rope(k)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        return lin(torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(-1, D), p + ".to_out.0")

    half = cfg.freq_dim // 2
    ang = t * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    c = "condition_embedder."
    temb = lin(F.silu(lin(torch.cat([ang.cos(), ang.sin()]), c + "time_embedder.linear_1")), c + "time_embedder.linear_2")
    tproj = lin(F.silu(temb), c + "time_proj").view(6, D)
    e = lin(F.gelu(lin(ctx, c + "text_embedder.linear_1"), approximate="tanh"), c + "text_embedder.linear_2")
    for i in range(cfg.num_layers):
        p = f"blocks.{i}"
        m = w[p + ".scale_shift_table"][0] + tproj
        x = x + attn(ln(x) * (1 + m[1]) + m[0], ln(x) * (1 + m[1]) + m[0], p + ".attn1", True) * m[2]
        x = x + attn(F.layer_norm(x, (D,), w[p + ".norm2.weight"], w[p + ".norm2.bias"], 1e-6), e, p + ".attn2", False)
        hh = ln(x) * (1 + m[4]) + m[3]
        x = x + lin(F.gelu(lin(hh, p + ".ffn.net.0.proj"), approximate="tanh"), p + ".ffn.net.2") * m[5]
    m = w["scale_shift_table"][0] + temb
    o = lin(ln(x) * (1 + m[1]) + m[0], "proj_out").view(f, h, ww, 1, 2, 2, C)
    return o.permute(6, 0, 3, 1, 4, 2, 5).reshape(C, Fr, H, Wd)


def test_dit_matches_direct_restatement():
    w = W.random_wan_weights(CFG, seed=1, std=0.15)
    g = torch.Generator().manual_seed(2)
    z, ctx, t = torch.randn(1, 4, 3, 4, 6, generator=g), torch.randn(1, 5, 10, generator=g), torch.tensor([730.0])
    out = W.WanDiT(CFG, w).forward(z, t, ctx)
    ref = _direct(w, CFG, z[0], t[0], ctx[0])
    assert out.shape == z.shape and ref.abs().max() > 0.05
    assert (out[0] - ref).abs().max().item() < 2e-4 * max(1.0, ref.abs().max().item())
    assert W.WanConfig().rope_axes == (44, 42, 42) and W.WanConfig().dim == 5120
