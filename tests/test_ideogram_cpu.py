"""Ideogram 4: the single-stream DiT against an independent restatement (explicit softmax attention, three-axis
rotary written per frequency), the logit-normal schedule's published values, packing layout, turbo adapter merge and
provider conformance."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_ideogram as X

CFG = X.IdeogramConfig(emb_dim=32, num_layers=2, num_heads=2, mlp_dim=48, adaln_dim=12, in_channels=8, llm_features_dim=26,
                       mrope_section=(4, 2, 2))


def _direct(w, cfg, llm, x, t, pos, ind):
    E, nh, hd = cfg.emb_dim, cfg.num_heads, cfg.head_dim
    lin = lambda v, n: v @ w[n + ".weight"].t() + (w[n + ".bias"] if n + ".bias" in w else 0)      # noqa: E731
    rms = lambda v, k, eps: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w[k]           # noqa: E731
    S = x.shape[0]
    half = hd // 2
    # rotary: frequency d uses axis 1 if d%3==1 (d < 3*sec1), axis 2 if d%3==2 (d < 3*sec2), else axis 0
    cos, sin = torch.zeros(S, half), torch.zeros(S, half)
    for s in range(S):
        for d in range(half):
            ax = 1 if (d % 3 == 1 and d < 3 * cfg.mrope_section[1]) else (2 if (d % 3 == 2 and d < 3 * cfg.mrope_section[2]) else 0)
            a = float(pos[s, ax]) * cfg.rope_theta ** (-2.0 * d / hd)
            cos[s, d], sin[s, d] = math.cos(a), math.sin(a)

    def rot(v):                                    # [S, nh, hd], pairs (i, i + half)
        a, b = v[..., :half], v[..., half:]
        return torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None]], -1)

    is_img, is_txt = (ind == 2).float()[:, None], (ind == 3).float()[:, None]
    h = lin(x * is_img, "input_proj") * is_img
    hh = E // 2
    f = torch.exp(-math.log(1e4) / (hh - 1) * torch.arange(hh).float())
    te = torch.cat([torch.sin(t * 1e4 * f), torch.cos(t * 1e4 * f)])
    cond = lin(F.silu(lin(te, "t_embedding.mlp_in")), "t_embedding.mlp_out")
    ada = F.silu(lin(cond, "adaln_proj"))
    h = h + lin(rms(llm * is_txt, "llm_cond_norm.weight", 1e-6), "llm_cond_proj") * is_txt
    h = h + w["embed_image_indicator.weight"][(ind == 2).long()]
    for i in range(cfg.num_layers):
        p = f"layers.{i}"
        sa, ga, sm, gm = lin(ada, p + ".adaln_modulation").chunk(4)
        n = rms(h, p + ".attention_norm1.weight", cfg.norm_eps) * (1 + sa)
        qkv = lin(n, p + ".attention.qkv").view(S, 3, nh, hd)
        q = rot(rms(qkv[:, 0], p + ".attention.norm_q.weight", 1e-5))
        k = rot(rms(qkv[:, 1], p + ".attention.norm_k.weight", 1e-5))
        sc = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        o = torch.einsum("hqk,khd->qhd", sc.softmax(-1), qkv[:, 2]).reshape(S, E)
        h = h + torch.tanh(ga) * rms(lin(o, p + ".attention.o"), p + ".attention_norm2.weight", cfg.norm_eps)
        n = rms(h, p + ".ffn_norm1.weight", cfg.norm_eps) * (1 + sm)
        ff = lin(F.silu(lin(n, p + ".feed_forward.w1")) * lin(n, p + ".feed_forward.w3"), p + ".feed_forward.w2")
        h = h + torch.tanh(gm) * rms(ff, p + ".ffn_norm2.weight", cfg.norm_eps)
    scale = 1 + lin(F.silu(ada), "final_layer.adaln_modulation")
    return lin(F.layer_norm(h, (E,), eps=1e-6) * scale, "final_layer.linear")


def test_dit_matches_restatement():
    torch.manual_seed(0)
    w = X.random_ideogram_weights(CFG, seed=3, std=0.2)
    model = X.IdeogramDiT(CFG, w)
    nt, gh, gw = 5, 2, 3
    pos, ind = X.packing(nt, gh, gw)
    S = nt + gh * gw
    llm, x = torch.randn(1, S, 26), torch.randn(1, S, 8)
    llm[:, nt:] = 0
    x[:, :nt] = 0
    t = torch.tensor([0.37])
    got = model.forward(llm, x, t, pos, ind)
    want = _direct(w, CFG, llm[0], x[0], t[0], pos, ind)
    assert got.shape == (1, S, 8) and torch.allclose(got[0], want, atol=3e-4, rtol=1e-3), (got[0] - want).abs().max()
    # a segment split changes the output; a uniform segment vector does not
    same = model.forward(llm, x, t, pos, ind, torch.zeros(S, dtype=torch.long))
    assert torch.allclose(same, got, atol=1e-6)
    seg = torch.cat([torch.zeros(nt, dtype=torch.long), torch.ones(gh * gw, dtype=torch.long)])
    assert not torch.allclose(model.forward(llm, x, t, pos, ind, seg), got, atol=1e-4)


def test_packing_and_full_size_config():
    pos, ind = X.packing(2, 2, 2)
    assert ind.tolist() == [3, 3, 2, 2, 2, 2]
    o = X.IMAGE_POSITION_OFFSET
    assert pos.tolist() == [[0, 0, 0], [1, 1, 1], [o, o, o], [o, o, o + 1], [o, o + 1, o], [o, o + 1, o + 1]]
    full = X.IdeogramConfig()
    assert full.head_dim == 256 and full.llm_features_dim == 13 * 4096 and sum(full.mrope_section) * 2 == 128
    cos, _ = X.mrope_tables(torch.tensor([[0.0, 1.0, 2.0]]), 256, full.rope_theta, full.mrope_section)
    inv = lambda d: full.rope_theta ** (-2.0 * d / 256)       # noqa: E731
    assert abs(cos[0, 0].item() - 1.0) < 1e-7                                      # d = 0 -> first axis (position 0)
    assert abs(cos[0, 1].item() - math.cos(1.0 * inv(1))) < 1e-6                   # d = 1 -> row axis
    assert abs(cos[0, 2].item() - math.cos(2.0 * inv(2))) < 1e-6                   # d = 2 -> column axis
    assert abs(cos[0, 61].item() - 1.0) < 1e-7 and abs(cos[0, 127].item() - 1.0) < 1e-7   # past 3 * 20 -> first axis


def test_schedule_matches_reference_golden_values():
    want = [0.99944723, 0.70425373, 0.54813725, 0.38193515, 0.00012339]
    for u, w in zip([0.0, 0.25, 0.5, 0.75, 1.0], want):
        assert abs(X.logit_normal_time(u, 256, 256, 0.5, 1.0) - w) < 1e-5
    assert X.preset_mu_std(8) == (0.5, 1.75) and X.preset_mu_std(20) == (0.0, 1.75) and X.preset_mu_std(48) == (0.0, 1.5)
    assert abs(X._ndtri(0.975) - 1.959964) < 1e-5 and abs(X._ndtri(0.001) + 3.090232) < 1e-5


def test_ideogram_providers_conform(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import ideogram as P
    from inference_b200.media import provider_registry
    from inference_b200.testkit import generator as kit

    snap = P.write_synthetic_snapshot(tmp_path / "ig")
    reg = provider_registry("cpu")
    assert sorted(i for i in reg.ids() if "ideogram" in i) == ["cpu_ideogram_4", "cpu_ideogram_4_turbo"]
    assert reg.descriptor_conformance_errors() == []
    q = reg.load("cpu_ideogram_4", LoadSpec.from_dir(snap))
    d = q.descriptor()
    assert d.capabilities.supports_guidance and not d.capabilities.supports_negative_prompt and d.capabilities.samplers == []
    kit.conformance(q, kit.Profile(steps=4, cancel_steps=6))
    kit.registry_conformance(reg, "cpu_ideogram_4", LoadSpec.from_dir(snap))
    turbo = reg.load("cpu_ideogram_4_turbo", LoadSpec.from_dir(snap))
    assert not turbo.descriptor().capabilities.supports_guidance
    kit.conformance(turbo, kit.Profile(steps=2, cancel_steps=5))
    # sigma table: framework sigma = 1 - model time, strictly decreasing from ~1 to ~0; polish steps use guidance 3
    s = q.pipe.native_sigmas(48, GenerationRequest(prompt="x", width=512, height=512))
    assert len(s) == 49 and s[0] > 0.999 and s[-1] < 0.01 and all(a > b for a, b in zip(s, s[1:]))
    assert [q.pipe.step_guidance(i, 48, 7.0) for i in (0, 44, 45, 47)] == [7.0, 7.0, 3.0, 3.0]
    # the turbo adapter changes the conditional network; guidance changes the quality render
    heavy_q, heavy_t = q.pipe.load_heavy(), turbo.pipe.load_heavy()
    k = "layers.0.attention.qkv.weight"
    assert heavy_t.uncond is None and heavy_q.uncond is not None
    assert not torch.equal(heavy_q.dit.bag[k], heavy_t.dit.bag[k])
    assert torch.equal(heavy_q.dit.bag["layers.0.attention.o.weight"], heavy_t.dit.bag["layers.0.attention.o.weight"])
    req = dict(prompt="a red kite", width=256, height=256, steps=4, seed=5)
    a = q.generate(GenerationRequest(**req, guidance=7.0)).images[0].pixels
    b = q.generate(GenerationRequest(**req, guidance=2.0)).images[0].pixels
    assert a != b
    with pytest.raises(InferenceError):
        q.generate(GenerationRequest(**{**req, "width": 250}))
    n = P.normalise_lora({"model.a.b.lora_up": torch.zeros(1), "x.lora_A.weight": torch.zeros(1)})
    assert set(n) == {"transformer.a.b.lora_B.weight", "transformer.x.lora_A.weight"}
