"""PiD: registry, position tables against explicit loops, the network (v1.0 and v1.5 adapter) against a heads-first
restatement, tiling and blending, the memory planner, the student sampler, caption selection and the engine end to end."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.media import pid as P

TINY = dict(num_groups=2, hidden_size=128, pixel_hidden_size=8, pixel_attn_hidden_size=128, pixel_num_groups=2, patch_depth=3,
            pixel_depth=1, patch_size=4, txt_embed_dim=32, txt_max_length=12, rope_ref_h=32, rope_ref_w=32, lq_latent_channels=4,
            lq_hidden_dim=16, lq_num_res_blocks=1, lq_interval=2, sr_scale=2, latent_spatial_down_factor=8)


def test_registry_and_configs():
    assert P.lookup("zimage-turbo") is P.SPECS["flux"] and P.lookup("flux2-klein-9b").latent_channels == 128
    assert P.lookup("qwenimage").ckpt_2k is None and P.lookup("sdxl").vp_frame and P.lookup("sd3").latent_norm == ("affine", 1.5305, 0.0609)
    assert P.lookup("flux2").latent_spatial_down_factor == 16 and P.lookup("wan") is None
    c = P.PidConfig.sr4x()
    assert (c.head_dim, c.pixel_head_dim, c.num_lq_outputs) == (64, 72, 7)
    v = P.PidConfig.sr4x_v1pt5()
    assert (v.rope_ref_h, v.lq_hidden_dim, v.lq_replicate_padding, v.pit_lq_inject) == (2048, 1024, True, True)
    got = P.config_for_spec(P.lookup("flux2"), True)
    assert (got.lq_latent_channels, got.latent_spatial_down_factor, got.sr_scale, got.pit_lq_inject) == (128, 16, 4, True)


def test_position_tables_match_explicit_loops():
    cos, sin = P.rope_2d_ntk(16, 3, 5, 2, 2)
    d_axis = 8.0
    ntk = d_axis / (d_axis - 2.0)
    th_h, th_w = 10000.0 * (3 / 2) ** ntk, 10000.0 * (5 / 2) ** ntk
    for r in range(3):
        for c in range(5):
            for m in range(8):
                j = m // 2
                a = (c * 16.0 / 4) / th_w ** (4 * j / 16) if m % 2 == 0 else (r * 16.0 / 2) / th_h ** (4 * j / 16)
                assert abs(cos[r * 5 + c, m].item() - math.cos(a)) < 1e-6 and abs(sin[r * 5 + c, m].item() - math.sin(a)) < 1e-6
    assert torch.all(P.rope_2d_ntk(8, 1, 1, 4, 4)[0] == 1.0)                     # a single cell sits at position 0
    ct, st = P.rope_1d_text(8, 4, 10000.0)
    assert abs(ct[3, 1].item() - math.cos(3 / 10000 ** (2 / 8))) < 1e-6 and st[0].abs().max() == 0
    pos = P.sincos_2d_pos(8, 2, 3)
    om = [1.0, 1.0 / 10000 ** 0.5]
    for i in range(2):
        for j in range(3):
            want = [math.sin(j * om[0]), math.sin(j * om[1]), math.cos(j * om[0]), math.cos(j * om[1]),
                    math.sin(i * om[0]), math.sin(i * om[1]), math.cos(i * om[0]), math.cos(i * om[1])]
            assert torch.allclose(pos[i * 3 + j], torch.tensor(want), atol=1e-6)
    x = torch.arange(2 * 3 * 8 * 12, dtype=torch.float32).view(2, 3, 8, 12)
    u = P.unfold_patches(x, 4)
    assert u.shape == (2, 6, 48) and torch.equal(u[0, 1].view(3, 4, 4), x[0, :, :4, 4:8])
    back = P.fold_patches(u.view(2, 6, 3, 16).permute(0, 2, 3, 1), 3, 2, 3, 4)
    assert torch.equal(back, x)


def _restated(cfg, w, x, t, y, lq, sigma):
    lin = lambda v, p: F.linear(v, w[p + ".weight"], w.get(p + ".bias"))                    # noqa: E731
    rms = lambda v, g: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * g          # noqa: E731
    H, P_, pd = cfg.hidden_size, cfg.patch_size, cfg.pixel_hidden_size
    B, _, Hh, Ww = x.shape
    hs, ws = Hh // P_, Ww // P_
    L = hs * ws

    def conv(v, p):
        if cfg.lq_replicate_padding:
            v = F.pad(v, (1, 1, 1, 1), mode="replicate")
            return F.conv2d(v, w[p + ".weight"], w[p + ".bias"])
        return F.conv2d(v, w[p + ".weight"], w[p + ".bias"], padding=1)

    z = lq
    proj_in = w["lq_proj.latent_proj.0.weight"].shape[1]
    f = int(round(math.sqrt(cfg.lq_latent_channels // proj_in)))
    if f > 1:
        b_, c_, h_, w_ = z.shape
        z = z.reshape(b_, c_ // (f * f), f, f, h_, w_).permute(0, 1, 4, 2, 5, 3).reshape(b_, c_ // (f * f), h_ * f, w_ * f)
    r = max((cfg.sr_scale * cfg.latent_spatial_down_factor) // (P_ * f), 1)
    z = z.repeat_interleave(r, 2).repeat_interleave(r, 3)
    z = conv(F.silu(conv(z, "lq_proj.latent_proj.0")), "lq_proj.latent_proj.2")
    for i in range(cfg.lq_num_res_blocks):
        q = f"lq_proj.latent_proj.{i + 3}.block"
        gn = lambda v, p: F.group_norm(v, 4, w[p + ".weight"], w[p + ".bias"], 1e-5)       # noqa: E731
        h = conv(F.silu(gn(z, q + ".0")), q + ".2")
        z = z + conv(F.silu(gn(h, q + ".3")), q + ".5")
    tok = z.flatten(2).transpose(1, 2)
    feats = [lin(tok, f"lq_proj.output_heads.{i}") for i in range(cfg.num_lq_outputs)]

    def gate(p, a, b_):
        return a + torch.sigmoid(lin(torch.cat([a, b_], -1), p + ".content_proj") - sigma.view(-1, 1, 1) * w[p + ".log_alpha"].exp()) * b_

    half = 128
    fr = torch.exp(-math.log(10.0) * torch.arange(half, dtype=torch.float32) / half)
    emb = torch.cat([(t[:, None] * fr).cos(), (t[:, None] * fr).sin()], 1)
    temb = lin(F.silu(lin(emb, "t_embedder.mlp.0")), "t_embedder.mlp.2").view(B, 1, H)
    ltxt = min(y.shape[1], cfg.txt_max_length)
    yv = rms(lin(y[:, :ltxt], "y_embedder.proj"), w["y_embedder.norm.weight"]) + w["y_pos_embedding"][:, :ltxt]
    cond = F.silu(temb)
    ci, si = P.rope_2d_ntk(cfg.head_dim, hs, ws, cfg.rope_ref_h // P_, cfg.rope_ref_w // P_)
    ct, st = P.rope_1d_text(cfg.head_dim, ltxt, cfg.text_rope_theta)

    def rope(v, c, s_):                                # [B, h, S, D] adjacent pairs
        a, b_ = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * c - b_ * s_, b_ * c + a * s_], -1).flatten(-2)

    def split(v, heads):
        q, k, vv = v.view(v.shape[0], v.shape[1], 3, heads, -1).unbind(2)
        return q.transpose(1, 2), k.transpose(1, 2), vv.transpose(1, 2)

    def sdpa(q, k, v):
        o = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(q.shape[-1]), -1) @ v
        return o.transpose(1, 2).flatten(2)

    s = rms(lin(P.unfold_patches(x, P_), "s_embedder.proj"), w["s_embedder.norm.weight"])
    for i in range(cfg.patch_depth):
        if i % cfg.lq_interval == 0 and i // cfg.lq_interval < len(feats):
            s = gate(f"lq_proj.gate_modules.{i // cfg.lq_interval}", s, feats[i // cfg.lq_interval])
        b_ = f"patch_blocks.{i}"
        mx, my = lin(cond, b_ + ".adaLN_modulation_img.0").chunk(6, -1), lin(cond, b_ + ".adaLN_modulation_txt.0").chunk(6, -1)
        xn = rms(s, w[b_ + ".norm_x1.weight"]) * (1 + mx[1]) + mx[0]
        yn = rms(yv, w[b_ + ".norm_y1.weight"]) * (1 + my[1]) + my[0]
        a = b_ + ".attn"
        qx, kx, vx = split(lin(xn, a + ".qkv_x"), cfg.num_groups)
        qy, ky, vy = split(lin(yn, a + ".qkv_y"), cfg.num_groups)
        qx, kx = rope(rms(qx, w[a + ".q_norm_x.weight"]), ci, si), rope(rms(kx, w[a + ".k_norm_x.weight"]), ci, si)
        qy, ky = rope(rms(qy, w[a + ".q_norm_y.weight"]), ct, st), rope(rms(ky, w[a + ".k_norm_y.weight"]), ct, st)
        o = sdpa(torch.cat([qy, qx], 2), torch.cat([ky, kx], 2), torch.cat([vy, vx], 2))
        s = s + lin(o[:, ltxt:], a + ".proj_x") * mx[2]
        yv = yv + lin(o[:, :ltxt], a + ".proj_y") * my[2]
        ffn = lambda v, p: F.linear(F.silu(F.linear(v, w[p + ".w1.weight"])) * F.linear(v, w[p + ".w3.weight"]), w[p + ".w2.weight"])   # noqa: E731
        s = s + ffn(rms(s, w[b_ + ".norm_x2.weight"]) * (1 + mx[4]) + mx[3], b_ + ".mlp_x") * mx[5]
        yv = yv + ffn(rms(yv, w[b_ + ".norm_y2.weight"]) * (1 + my[4]) + my[3], b_ + ".mlp_y") * my[5]
    s = F.silu(s + temb)
    if cfg.pit_lq_inject:
        s = gate("pit_lq_gate", s, lin(tok, "lq_proj.pit_head"))
    sc = s.reshape(B * L, H)
    p2 = P_ * P_
    xp = lin(x.permute(0, 2, 3, 1), "pixel_embedder.proj") + P.sincos_2d_pos(pd, Hh, Ww).view(1, Hh, Ww, pd)
    xp = xp.reshape(B, hs, P_, ws, P_, pd).permute(0, 1, 3, 2, 4, 5).reshape(B * L, p2, pd)
    cp, sp = P.rope_2d_ntk(cfg.pixel_head_dim, hs, ws, cfg.rope_ref_h // P_, cfg.rope_ref_w // P_)
    for i in range(cfg.pixel_depth):
        b_ = f"pixel_blocks.{i}"
        m = lin(sc, b_ + ".adaLN_modulation.0").view(B * L, p2, 6 * pd).chunk(6, -1)
        h = (rms(xp, w[b_ + ".norm1.weight"]) * (1 + m[1]) + m[0]).reshape(B * L, p2 * pd)
        hc = lin(h, b_ + ".compress_to_attn").view(B, L, -1)
        q, k, v = split(lin(hc, b_ + ".attn.qkv"), cfg.pixel_num_groups)
        q, k = rope(rms(q, w[b_ + ".attn.q_norm.weight"]), cp, sp), rope(rms(k, w[b_ + ".attn.k_norm.weight"]), cp, sp)
        a = lin(lin(sdpa(q, k, v), b_ + ".attn.proj").reshape(B * L, -1), b_ + ".expand_from_attn").view(B * L, p2, pd)
        xp = xp + a * m[2]
        h = rms(xp, w[b_ + ".norm2.weight"]) * (1 + m[4]) + m[3]
        xp = xp + lin(F.gelu(lin(h, b_ + ".mlp.fc1")), b_ + ".mlp.fc2") * m[5]
    out = lin(rms(xp, w["final_layer.norm.weight"]), "final_layer.linear").reshape(B, L, p2, 3).permute(0, 3, 2, 1)
    return P.fold_patches(out, 3, hs, ws, P_)


@pytest.mark.parametrize("v15,proj_in", [(False, None), (True, None), (True, 1)])
def test_network_matches_restatement(v15, proj_in):
    cfg = P.PidConfig(**TINY, lq_replicate_padding=v15, pit_lq_inject=v15)
    w = P.random_pid_weights(cfg, seed=1, proj_in=proj_in)
    assert P.detect_v1pt5(w) == v15
    net = P.PidNet(w, cfg)
    assert net.unpatchify == (2 if proj_in == 1 else 1) and net.upsample == (2 if proj_in == 1 else 4)
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(2, 3, 16, 32, generator=g), torch.randn(2, 14, 32, generator=g)
    lq, t, sig = torch.randn(2, 4, 1, 2, generator=g), torch.tensor([866.0, 342.0]), torch.tensor([0.0, 0.4])
    got = net.forward(x, t, y, lq, sig)
    want = _restated(cfg, w, x, t, y, lq, sig)
    assert got.shape == (2, 3, 16, 32) and torch.allclose(got, want, atol=3e-5, rtol=1e-4)
    assert not torch.allclose(net.forward(x, t, y, lq * 0, sig), got, atol=1e-4)            # the latent really conditions
    assert not torch.allclose(net.forward(x, t, y, lq, sig + 5.0), got, atol=1e-5)          # and the gates see sigma
    from inference_b200.contracts.errors import LoadError
    with pytest.raises(LoadError):
        P.detect_v1pt5({k: v for k, v in w.items() if not k.startswith("lq_proj.gate_modules.")})
    mixed = dict(w)
    if v15:
        mixed.pop("pit_lq_gate.content_proj.weight")
    else:
        mixed["pit_lq_gate.content_proj.weight"] = torch.zeros(1, 4)
    with pytest.raises(LoadError):
        P.detect_v1pt5(mixed)


def test_tiling_and_blending():
    ax = P.tile_axis(4096, 2048, 256)
    assert ax[0][0] == 0 and ax[-1][1] == 4096 and all(e - s == 2048 for s, e in ax) and all(b[0] < a[1] for a, b in zip(ax, ax[1:]))
    assert P.tile_axis(100, 128, 16) == [(0, 100)] and P.tile_axis(300, 128, 0) == [(0, 128), (128, 256), (172, 300)]
    plan = P.plan_tiles(96, 64, 50, 20, 16)                         # tile / overlap snap to the 16-pixel latent cell
    assert all((y1 - y0) == 48 and (x1 - x0) == 48 and y0 % 16 == 0 and x0 % 16 == 0 for y0, y1, x0, x1 in plan)
    assert len(plan) == len(P.tile_axis(96, 48, 16)) * len(P.tile_axis(64, 48, 16))
    r = P.axis_ramp(10, True, True, 3)
    assert r[0] == pytest.approx(0.25) and r[2] == pytest.approx(0.75) and torch.all(r[3:7] == 1.0) and r[-1] == pytest.approx(0.25)
    assert torch.all(P.axis_ramp(10, False, False, 3) == 1.0)

    class Net:                                           # a pointwise map: tiling must reproduce it exactly
        calls = 0

        def forward(self, x, t, y, lq, sigma):
            Net.calls += 1
            assert lq.shape[2] * 8 == x.shape[2] and lq.shape[3] * 8 == x.shape[3]
            return x * 2.0 + F.interpolate(lq[:, :3], scale_factor=8, mode="nearest")
    x, lq = torch.randn(1, 3, 48, 64), torch.randn(1, 4, 6, 8)
    whole = Net().forward(x, None, None, lq, None)
    Net.calls = 0
    tiled = P.forward_tiled(Net(), x, None, None, lq, None, 32, 16)
    assert Net.calls == len(P.plan_tiles(48, 64, 32, 16, 8)) > 1 and torch.allclose(tiled, whole, atol=1e-5)
    Net.calls = 0
    P.forward_tiled(Net(), x, None, None, lq, None, 128, 16)
    assert Net.calls == 1


def test_memory_planner():
    base, dbl = P.estimated_decode_peak_gib(1, 512, 512, 16, 1536), P.estimated_decode_peak_gib(1, 1024, 1024, 16, 1536)
    assert abs(dbl - 4 * base) / base < 1e-9
    whole, tiled = P.estimated_decode_peak_gib(1, 6144, 6144, 16, 1536), P.tiled_peak_gib(1, 6144, 6144, 2048, 16, 1536)
    assert tiled < 0.5 * whole and tiled > P.resident_full_gib(1, 6144, 6144)
    assert P.plan_tile_edge(1, 6144, 6144, 16, 1536, 100.0) == (6144, 256, True)
    edge, ov, fits = P.plan_tile_edge(1, 6144, 6144, 16, 1536, 8.0)
    assert not fits and ov == 256 and edge % 512 == 0 and 1024 <= edge <= 2048
    from inference_b200.contracts.errors import InferenceError
    P.guard("m", 1, 1024, 1024, 4, P.PidConfig.sr4x(), 24.0)
    with pytest.raises(InferenceError):
        P.guard("m", 4, 4096, 4096, 4, P.PidConfig.sr4x(), 8.0)


def test_sampler():
    s = P.Sampler()
    assert s.steps == 4 and s.num_eps == 3 and P.Sampler(sde=False).num_eps == 0
    noise, eps = s.draws(7, 1, 4, 6)
    assert noise.shape == (1, 3, 4, 6) and len(eps) == 3 and not torch.equal(eps[0], eps[1]) and torch.equal(s.draws(7, 1, 4, 6)[0], noise)
    seen = []

    def perfect(x, t):                                   # the exact velocity towards a known clean image
        seen.append(float(t[0]))
        return (x - clean) / (seen[-1] / 1000.0)
    clean = torch.rand(1, 3, 4, 6) * 1.6 - 0.8
    out = s.run(perfect, noise, eps)
    assert torch.allclose(out, clean, atol=1e-4) and seen == pytest.approx([999.0, 866.0, 634.0, 342.0])
    ode = P.Sampler(t_list=(1.0, 0.5, 0.0), sde=False)
    assert torch.allclose(ode.run(lambda x, t: torch.ones_like(x), torch.zeros(1, 3, 2, 2), []), torch.full((1, 3, 2, 2), -1.0))
    assert s.run(lambda x, t: -x * 100, noise, eps).abs().max() <= 1.0           # clamped
    from inference_b200.contracts.errors import Canceled
    with pytest.raises(Canceled):
        s.run(perfect, noise, eps, cancel=lambda: True)


def _write_gemma(d):
    import tokenizers
    from tokenizers import decoders, models, pre_tokenizers, trainers

    from inference_b200.io.safetensors_io import save_file
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import random_llama_weights

    d.mkdir()
    tok = tokenizers.Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.train_from_iterator([P.CHI_PROMPT, "a red fox jumps over the lazy dog"], trainers.BpeTrainer(
        vocab_size=300, special_tokens=["<pad>", "<bos>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    tok.save(str(d / "tokenizer.json"))
    cj = {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "vocab_size": tok.get_vocab_size(), "hidden_size": 32,
          "intermediate_size": 64, "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
          "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 8192, "sliding_window": 4096,
          "query_pre_attn_scalar": 16, "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0}
    (d / "config.json").write_text(json.dumps(cj))
    save_file(random_llama_weights(ModelConfig.from_json(cj), 3, std=0.1), d / "model.safetensors")


def test_caption_and_engine_end_to_end(tmp_path, monkeypatch):
    from inference_b200.contracts.errors import LoadError

    assert P.CHI_PROMPT.startswith("Given a user prompt") and P.CHI_PROMPT.endswith("User Prompt: ")
    monkeypatch.setattr(P, "CHI_PROMPT", "Enhance the prompt. User Prompt: ")       # a short prefix keeps the toy encoder quick
    from inference_b200.io.safetensors_io import save_file

    assert P.select_index(555) == [0] + list(range(256, 555)) and len(P.select_index(555)) == 300
    _write_gemma(tmp_path / "gemma")
    enc = P.CaptionEncoder(tmp_path / "gemma")
    ids, real = enc.token_ids("a red fox")
    assert len(ids) == enc.num_chi_tokens + 298 and real < len(ids) and all(i == P.PAD_ID for i in ids[real:])
    e1, e2 = enc.encode("a red fox"), enc.encode("a lazy dog")
    assert e1.shape == (1, 300, 32) and torch.isfinite(e1).all() and not torch.allclose(e1, e2) and torch.equal(e1, enc.encode("a red fox"))
    assert torch.allclose(e1[:, 0], e2[:, 0], atol=1e-6)                        # position 0 only ever sees the first token
    cfg = P.PidConfig(**{**TINY, "txt_embed_dim": 32, "txt_max_length": 300})
    save_file(P.random_pid_weights(cfg, seed=2), tmp_path / "pid.safetensors")
    with pytest.raises(LoadError):
        P.PidEngine.load(tmp_path / "pid.safetensors", tmp_path / "gemma", "wan", "cpu")
    with pytest.raises(LoadError):
        P.PidEngine.load(tmp_path / "nope.safetensors", tmp_path / "gemma", "sdxl", "cpu")
    eng = P.PidEngine.load(tmp_path / "pid.safetensors", tmp_path / "gemma", "sdxl", "cpu", base_cfg=cfg)
    assert (eng.scale, eng.vae_compression, eng.cfg.lq_latent_channels, eng.cfg.pit_lq_inject) == (4, 8, 4, False)
    dec = eng.decoder("a red fox", 0.0, seed=5)
    z = torch.randn(1, 4, 1, 2, generator=torch.Generator().manual_seed(0))
    img = dec.decode(z)
    assert img.shape == (1, 3, 32, 64) and img.abs().max() <= 1.0 and torch.equal(img, eng.decoder("a red fox", 0.0, seed=5).decode(z))
    assert not torch.equal(img, eng.decoder("a red fox", 0.0, seed=6).decode(z))
    assert not torch.equal(img, eng.decoder("a lazy dog", 0.0, seed=5).decode(z))
    assert not torch.equal(img, eng.decoder("a red fox", 0.5, seed=5).decode(z))
    assert eng.decoder("x", 0.0, 1, latent_hw=(1, 2), safe_gib=100.0).tile is None
    assert eng.decoder("x", 0.0, 1, latent_hw=(192, 192), safe_gib=8.0).tile == (P.plan_tile_edge(1, 6144, 6144, 4, 128, 8.0)[0], 256)
    # early-stop capture: hand a still-noisy latent to the decoder at the first schedule point at / below the ceiling
    sig = [1.0, 0.8, 0.5, 0.2, 0.0]
    assert P.flow_capture_for_request(True, 0.6, sig, 0) == (0.5, 3)
    assert P.flow_capture_for_request(False, 0.6, sig, 0) == (0.0, 5) and P.flow_capture_for_request(True, None, sig, 0) == (0.0, 5)
    assert P.flow_capture_for_request(True, 0.6, sig, 2) == (0.0, 5) and P.flow_capture_for_request(True, 0.1, sig, 0) == (0.0, 5)


def test_flux_generator_decodes_through_pid(tmp_path, monkeypatch):
    """`use_pid` on a FLUX generator loaded with the pixel decoder: same denoising, the latent goes to PiD instead of the
    VAE and the image comes back `scale` times larger; requests that do not ask for it never touch the decoder."""
    from inference_b200.contracts.errors import InferenceError, LoadError
    from inference_b200.contracts.gen_core import GenerationRequest
    from inference_b200.contracts.gen_core.runtime import LoadSpec, WeightsSource
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media import flux
    from inference_b200.media.catalog import provider_registry

    monkeypatch.setattr(P, "CHI_PROMPT", "Enhance the prompt. User Prompt: ")
    snap = flux.write_synthetic_snapshot(tmp_path / "flux", flux.Variant.SCHNELL)
    _write_gemma(tmp_path / "gemma")
    cfg = P.PidConfig(**{**TINY, "txt_embed_dim": 32, "txt_max_length": 300, "lq_latent_channels": 16, "sr_scale": 4, "patch_size": 16,
                         "patch_depth": 2, "rope_ref_h": 256, "rope_ref_w": 256})
    save_file(P.random_pid_weights(cfg, seed=2), tmp_path / "pid.safetensors")
    reg = provider_registry("cpu")
    plain_gen = reg.load("cpu_flux1_schnell", LoadSpec.from_dir(snap))
    req = lambda **kw: GenerationRequest(prompt="a red fox", width=256, height=256, steps=2, seed=5, **kw)      # noqa: E731
    with pytest.raises(InferenceError, match="no PiD decoder is loaded"):
        plain_gen.generate(req(use_pid=True))
    spec = LoadSpec.from_dir(snap)
    spec.pid = WeightsSource.file(tmp_path / "pid.safetensors")
    with pytest.raises(LoadError):
        reg.load("cpu_flux1_schnell", spec)                                # the caption encoder is missing
    spec.components["pid_gemma"] = WeightsSource.dir(tmp_path / "gemma")
    gen = reg.load("cpu_flux1_schnell", spec)
    import inference_b200.media.pid as pid_mod
    orig = pid_mod.PidEngine.load
    pid_mod.PidEngine.load = staticmethod(lambda ck, gd, bb, be="b200", base_cfg=None: orig(ck, gd, bb, be, cfg))   # the tiny topology
    try:
        base = gen.generate(req()).images[0]
        assert gen.pipe._pid_engine is None and base.pixels == plain_gen.generate(req()).images[0].pixels
        events = []
        big = gen.generate(req(use_pid=True), events.append).images[0]
        assert (big.width, big.height) == (1024, 1024) and len(big.pixels) == 1024 * 1024 * 3 and gen.pipe._pid_engine is not None
        assert gen.pipe._pid_engine.spec.latent_space == "flux" and len(events) == 3
        assert gen.generate(req(use_pid=True)).images[0].pixels == big.pixels
        with pytest.raises(InferenceError, match="pid_capture_sigma"):
            gen.generate(req(use_pid=True, pid_capture_sigma=0.3))
    finally:
        pid_mod.PidEngine.load = orig


def test_family_scaffolding_decodes_through_pid(tmp_path, monkeypatch):
    """The shared family pipeline: a family that names its PiD latent space (Krea: the Qwen-Image autoencoder's) accepts
    the decoder at load and routes `use_pid` requests through it; a family without one refuses the components."""
    from inference_b200.contracts.errors import InferenceError, Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest
    from inference_b200.contracts.gen_core.runtime import LoadSpec, WeightsSource
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media import krea, sana
    from inference_b200.media.catalog import provider_registry

    monkeypatch.setattr(P, "CHI_PROMPT", "Enhance the prompt. User Prompt: ")
    snap = krea.write_synthetic_snapshot(tmp_path / "krea")
    _write_gemma(tmp_path / "gemma")
    reg = provider_registry("cpu")
    plain = reg.load("cpu_krea_2_turbo", LoadSpec.from_dir(snap))
    ch = plain.pipe.latent_channels
    cfg = P.PidConfig(**{**TINY, "txt_embed_dim": 32, "txt_max_length": 300, "lq_latent_channels": ch, "sr_scale": 4, "patch_size": 16,
                         "patch_depth": 2, "rope_ref_h": 256, "rope_ref_w": 256})
    save_file(P.random_pid_weights(cfg, seed=2), tmp_path / "pid.safetensors")
    spec = LoadSpec.from_dir(snap)
    spec.pid = WeightsSource.file(tmp_path / "pid.safetensors")
    spec.components["pid_gemma"] = WeightsSource.dir(tmp_path / "gemma")
    gen = reg.load("cpu_krea_2_turbo", spec)
    orig = P.PidEngine.load
    monkeypatch.setattr(P.PidEngine, "load", staticmethod(lambda ck, gd, bb, be="b200", base_cfg=None: orig(ck, gd, bb, be, replace_channels(cfg, bb))))
    req = lambda **kw: GenerationRequest(prompt="a red fox", width=256, height=256, steps=2, seed=5, **kw)      # noqa: E731
    with pytest.raises(InferenceError, match="no PiD decoder is loaded"):
        plain.generate(req(use_pid=True))
    assert gen.generate(req()).images[0].pixels == plain.generate(req()).images[0].pixels and gen.pipe._pid_engine is None
    big = gen.generate(req(use_pid=True)).images[0]
    assert (big.width, big.height) == (1024, 1024) and gen.pipe._pid_engine.spec.latent_space == "qwenimage"
    with pytest.raises(InferenceError, match="pid_capture_sigma"):
        gen.generate(req(use_pid=True, pid_capture_sigma=0.3))
    other = LoadSpec.from_dir(sana.write_synthetic_snapshot(tmp_path / "sana"))
    other.pid = WeightsSource.file(tmp_path / "pid.safetensors")
    other.components["pid_gemma"] = WeightsSource.dir(tmp_path / "gemma")
    with pytest.raises(Unsupported):
        reg.load("cpu_" + sana.VARIANTS[0].id, other)


def replace_channels(cfg, backbone):
    from dataclasses import replace

    return replace(cfg, lq_latent_channels=P.lookup(backbone).latent_channels)
