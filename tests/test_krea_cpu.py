"""Krea 2: the DiT against an independent restatement (explicit softmax attention with repeated kv heads, complex
rotary, per-layer einsum projector), the sigma tables against the reference's golden values, the guidance rule, and
provider conformance on the oracle backend."""
import math

import torch
import torch.nn.functional as F

from inference_b200.models import dit_krea as K

CFG = K.KreaConfig(num_attention_heads=4, num_kv_heads=2, attention_head_dim=16, num_layers=2, intermediate_size=40,
                   axes_dims_rope=(4, 6, 6), num_text_layers=3, num_layerwise_text_blocks=1, num_refiner_text_blocks=1,
                   text_hidden_dim=32, text_intermediate_size=48, text_num_attention_heads=2, text_num_kv_heads=1,
                   in_channels=16)


def _rms1(x, scale, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (scale + 1.0)


def _direct(w, cfg, latent, sigma, context, refs=()):
    """One sample, written from the architecture description only."""
    hd, eps, H = cfg.attention_head_dim, cfg.norm_eps, cfg.hidden_size

    def lin(x, n):
        y = x @ w[n + ".weight"].t()
        return y + w[n + ".bias"] if n + ".bias" in w else y

    def attn(x, p, heads, kv, pos):
        S = x.shape[0]
        q = _rms1(lin(x, p + ".attn.to_q").view(S, heads, hd), w[p + ".attn.norm_q.weight"], eps)
        k = _rms1(lin(x, p + ".attn.to_k").view(S, kv, hd), w[p + ".attn.norm_k.weight"], eps)
        v = lin(x, p + ".attn.to_v").view(S, kv, hd)
        if pos is not None:
            ang = []
            for a, d in enumerate(cfg.axes_dims_rope):
                inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2).double() / d))
                ang.append(pos[:, a:a + 1].double() * inv)
            fr = torch.polar(torch.ones_like(torch.cat(ang, -1)), torch.cat(ang, -1))

            def rot(t):
                tc = torch.view_as_complex(t.double().reshape(*t.shape[:-1], -1, 2))
                return torch.view_as_real(tc * fr[:, None, :]).flatten(-2).float()
            q, k = rot(q), rot(k)
        k, v = k.repeat_interleave(heads // kv, 1), v.repeat_interleave(heads // kv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(hd)
        o = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(S, heads * hd)
        return lin(o * torch.sigmoid(lin(x, p + ".attn.to_gate")), p + ".attn.to_out.0")

    def mlp(x, p):
        return lin(F.silu(lin(x, p + ".ff.gate")) * lin(x, p + ".ff.up"), p + ".ff.down")

    def fusion(x, p):
        x = x + attn(_rms1(x, w[p + ".norm1.weight"], eps), p, cfg.text_num_attention_heads, cfg.text_num_kv_heads, None)
        return x + mlp(_rms1(x, w[p + ".norm2.weight"], eps), p)

    L, NL, D = context.shape
    toks = []
    for tkn in range(L):                                  # every token: a sequence over the layer axis
        h = context[tkn]
        for i in range(cfg.num_layerwise_text_blocks):
            h = fusion(h, f"text_fusion.layerwise_blocks.{i}")
        toks.append(torch.einsum("ld,l->d", h, w["text_fusion.projector.weight"][0]))
    c = torch.stack(toks)
    for i in range(cfg.num_refiner_text_blocks):
        c = fusion(c, f"text_fusion.refiner_blocks.{i}")
    c = lin(F.gelu(lin(_rms1(c, w["txt_in.norm.weight"], eps), "txt_in.linear_1")), "txt_in.linear_2")

    def embed(z):
        C, Hh, Ww = z.shape
        ht, wt = Hh // 2, Ww // 2
        rows = [z[:, 2 * i:2 * i + 2, 2 * j:2 * j + 2].reshape(-1) for i in range(ht) for j in range(wt)]
        return lin(torch.stack(rows), "img_in"), ht, wt

    img, ht, wt = embed(latent)
    ref_toks = [embed(r)[0] for r in refs]
    half = cfg.timestep_embed_dim // 2
    fq = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    te = torch.cat([torch.cos(sigma * 1000.0 * fq), torch.sin(sigma * 1000.0 * fq)])
    t = lin(F.gelu(lin(te, "time_embed.linear_1")), "time_embed.linear_2")
    tvec = lin(F.gelu(t), "time_mod_proj")
    grid = [(0.0, float(i), float(j)) for i in range(ht) for j in range(wt)]
    pos = [(0.0, 0.0, 0.0)] * L
    for r in range(len(refs)):
        pos += [(float(r + 1), a, b) for _, a, b in grid]
    pos = torch.tensor(pos + grid)
    x = torch.cat([c, *ref_toks, img])
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        m = tvec + w[p + ".scale_shift_table"].reshape(-1)
        prs, prh, prg, pos_s, pos_h, pos_g = m.chunk(6)
        x = x + prg * attn(_rms1(x, w[p + ".norm1.weight"], eps) * (1 + prs) + prh, p, cfg.num_attention_heads,
                           cfg.num_kv_heads, pos)
        x = x + pos_g * mlp(_rms1(x, w[p + ".norm2.weight"], eps) * (1 + pos_s) + pos_h, p)
    fm = t[None, :] + w["final_layer.scale_shift_table"]
    out = lin(_rms1(x, w["final_layer.norm.weight"], eps) * (1 + fm[0]) + fm[1], "final_layer.linear")
    out = out[L + len(refs) * ht * wt:]
    C = cfg.latent_channels
    z = torch.zeros(C, ht * 2, wt * 2)
    for n in range(ht * wt):
        i, j = divmod(n, wt)
        z[:, 2 * i:2 * i + 2, 2 * j:2 * j + 2] = out[n].view(C, 2, 2)
    return z


def test_dit_matches_restatement_t2i_and_edit():
    torch.manual_seed(0)
    w = K.random_krea_weights(CFG, seed=3, std=0.2)
    model = K.KreaDiT(CFG, w)
    latent = torch.randn(1, 4, 6, 8)
    ctx = torch.randn(1, 5, 3, 32)
    sig = torch.tensor([0.63])
    got = model.forward(latent, sig, ctx)
    want = _direct(w, CFG, latent[0], sig[0], ctx[0])
    assert got.shape == (1, 4, 6, 8)
    assert torch.allclose(got[0], want, atol=2e-4, rtol=1e-3), (got[0] - want).abs().max()
    refs = [torch.randn(1, 4, 6, 8), torch.randn(1, 4, 6, 8)]
    got_e = model.forward(latent, sig, ctx, refs=refs)
    want_e = _direct(w, CFG, latent[0], sig[0], ctx[0], [r[0] for r in refs])
    assert torch.allclose(got_e[0], want_e, atol=2e-4, rtol=1e-3)
    assert not torch.allclose(got_e, got, atol=1e-3)
    # the text branch can be hoisted out of the step loop
    fused = model.text_fusion(ctx)
    assert torch.allclose(model.forward(latent, sig, None, fused_context=fused), got, atol=1e-6)
    import pytest

    with pytest.raises(ValueError):
        model.forward(latent, sig, ctx, refs=[torch.randn(1, 4, 4, 8)])


def test_positions_and_config_validation():
    import pytest

    p = K.krea_positions(3, 2, 2, n_refs=1)
    assert p.shape == (3 + 8, 3) and p[:3].abs().sum() == 0
    assert p[3:7, 0].tolist() == [1.0] * 4 and p[7:, 0].tolist() == [0.0] * 4
    assert p[7:, 1:].tolist() == [[0, 0], [0, 1], [1, 0], [1, 1]]
    assert torch.equal(K.krea_positions(3, 2, 2, 0), torch.cat([p[:3], p[7:]]))
    with pytest.raises(ValueError):
        K.KreaConfig(axes_dims_rope=(32, 48, 40)).validate()
    full = K.KreaConfig()
    full.validate()
    assert full.hidden_size == 6144 and full.latent_channels == 16


def test_schedules_match_reference_golden_values():
    from inference_b200.media import krea as P

    want = [1.0, 0.95672369, 0.90453076, 0.84034878, 0.75951093, 0.65456682, 0.51284409, 0.31090108, 0.0]
    got = P.krea_sigmas(8, P.TURBO_MU)                    # candle-gen-krea/src/schedule.rs tests
    assert all(abs(a - b) < 1e-5 for a, b in zip(got, want)) and len(got) == 9
    assert abs(P.dynamic_mu(256.0) - 0.5) < 1e-9 and abs(P.dynamic_mu(6400.0) - 1.15) < 1e-9
    assert abs(P.dynamic_mu(4096.0) - 0.90625) < 1e-9
    want4 = [1.0, 0.88130659, 0.71223223, 0.45205718, 0.0]
    assert all(abs(a - b) < 1e-5 for a, b in zip(P.krea_sigmas(4, P.dynamic_mu(4096.0)), want4))
    assert P.krea_sigmas(1, P.TURBO_MU) == [1.0, 0.0]
    c, u = torch.tensor([2.0]), torch.tensor([1.0])
    assert P.krea_cfg_combine(c, u, 1.0).item() == 3.0      # offset by one: guidance 1 already extrapolates
    assert P.krea_cfg_combine(c, u, 0.0).item() == 2.0


def test_krea_providers_conform(tmp_path):
    import pytest

    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.krea import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "krea")
    reg = provider_registry("cpu")
    assert sorted(i for i in reg.ids() if "krea" in i) == ["cpu_krea_2_raw", "cpu_krea_2_turbo"]
    assert reg.descriptor_conformance_errors() == []
    turbo = reg.load("cpu_krea_2_turbo", LoadSpec.from_dir(snap))
    kit.conformance(turbo, kit.Profile(steps=2, cancel_steps=5))
    kit.registry_conformance(reg, "cpu_krea_2_turbo", LoadSpec.from_dir(snap))
    req = dict(prompt="a red fox", width=256, height=256, steps=2, seed=5)
    with pytest.raises(InferenceError):
        turbo.generate(GenerationRequest(**req, negative_prompt="blurry"))     # distilled: no negative prompt
    raw = reg.load("cpu_krea_2_raw", LoadSpec.from_dir(snap))
    a = raw.generate(GenerationRequest(**req, guidance=0.0)).images[0].pixels   # guidance 0: one forward per step
    b = raw.generate(GenerationRequest(**req)).images[0].pixels                 # default 3.5, empty negative
    c = raw.generate(GenerationRequest(**req, guidance=3.5, negative_prompt="")).images[0].pixels
    d = raw.generate(GenerationRequest(**req, sampler="heun", scheduler="simple")).images[0].pixels
    assert b == c and a != b and d != b and len(a) == 256 * 256 * 3


def test_krea_trainer(tmp_path):
    """LoRA / LoKr training on the Krea DiT: adapters on the attention q / k / v / out projections only, raw-sigma
    conditioning, raw velocity regressed towards eps - x0; a few steps lower the loss of the item they were trained on."""
    import json

    import torch

    from inference_b200.contracts.gen_core import LoadSpec, TrainingConfig
    from inference_b200.io.safetensors_io import load_file, save_file
    from inference_b200.media import provider_registry
    from inference_b200.media.krea import write_synthetic_snapshot
    from inference_b200.media.train import KREA_TARGETS
    from inference_b200.testkit.aux_suites import TrainerProfile, trainer_conformance

    snap = write_synthetic_snapshot(tmp_path / "krea")
    reg = provider_registry("cpu")
    assert "cpu_krea_lora_trainer" in reg.ids("trainer")
    tr = reg.load_kind("trainer", "cpu_krea_lora_trainer", LoadSpec.from_dir(snap))
    c = tr.cfg
    ds = tmp_path / "ds"
    ds.mkdir()
    g = torch.Generator().manual_seed(0)
    hw = 4 * c.patch_size
    for i in range(2):
        save_file({"latent": torch.randn(c.latent_channels, hw, hw, generator=g),
                   "txt": torch.randn(5, c.num_text_layers, c.text_hidden_dim, generator=g)}, ds / f"item{i}.safetensors")
    items = tr._items(ds)
    noise = torch.randn(c.latent_channels, hw, hw, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    final = tr.train(TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "run", steps=8, learning_rate=5e-3, rank=4, alpha=4.0, seed=3),
                     lambda p: None)
    ad = load_file(final)
    names = {k[len("transformer."):].split(".lora_")[0] for k in ad}
    assert names and all(n.endswith(KREA_TARGETS) for n in names) and not any("to_gate" in n or ".ff." in n for n in names)
    tr.model.lora = {k[len("transformer."):-len(".lora_A.weight")]: (ad[k], ad[k.replace("lora_A", "lora_B")], 1.0)
                     for k in ad if k.endswith("lora_A.weight")}
    assert float(tr.loss_on(items[0], 0.5, noise)) < before
    tr.model.lora = None
    assert float(tr.loss_on(items[0], 0.5, noise)) == before
    trainer_conformance(reg.load_kind("trainer", "cpu_krea_lora_trainer", LoadSpec.from_dir(snap)),
                        TrainerProfile(ds, tmp_path / "out", steps=3, rank=2))
    lokr = tr.train(TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "lokr", steps=2, learning_rate=5e-3, rank=2, alpha=2.0, seed=3,
                                   adapter="lokr"), lambda p: None)
    assert any(k.endswith("lokr_w1") for k in load_file(lokr))
