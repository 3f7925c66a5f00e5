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


def test_video_autoencoder_invariants():
    from inference_b200.models.vae_qwen import QwenVaeConfig, QwenVaeDecoder, WanVaeDecoder, random_wan_vae_weights

    cfg = QwenVaeConfig(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    w = random_wan_vae_weights(cfg, seed=3, std=0.2)
    dec = WanVaeDecoder(cfg, w)
    g = torch.Generator().manual_seed(1)
    z = torch.randn(1, 16, 3, 3, 4, generator=g)
    out = dec.decode(z)
    assert out.shape == (1, 3, 9, 24, 32)                                   # 1 + 4 * (3 - 1) frames
    # one latent frame is the image autoencoder
    torch.testing.assert_close(dec.decode(z[:, :, :1])[:, :, 0], QwenVaeDecoder(cfg, w).decode(z[:, :, 0]), atol=1e-5, rtol=1e-5)
    # causal in time: the frames that latent frames 0..k produce do not move when later latent frames change
    z2 = z.clone()
    z2[:, :, 2] = torch.randn(1, 16, 3, 4, generator=g)
    out2 = dec.decode(z2)
    torch.testing.assert_close(out2[:, :, :5], out[:, :, :5], atol=1e-5, rtol=1e-5)
    assert (out2[:, :, 5:] - out[:, :, 5:]).abs().max() > 1e-3
    torch.testing.assert_close(dec.decode(z[:, :, :2]), out[:, :, :5], atol=1e-5, rtol=1e-5)


def test_schedule_and_provider(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.wan import wan_sigmas, write_synthetic_snapshot

    s = wan_sigmas(40)
    assert len(s) == 41 and abs(s[0] - (1.0 - 1e-6)) < 1e-12 and s[-1] == 0.0 and all(a > b for a, b in zip(s, s[1:]))
    raw = 1.0 + (0.001 - 1.0) * 39 / 40
    assert abs(s[39] - 12 * raw / (1 + 11 * raw)) < 1e-12
    assert sum(1 for v in s[:-1] if v * 1000 >= 875) > 20                 # shift 12 keeps most steps on the high-noise expert
    snap = write_synthetic_snapshot(tmp_path / "wan")
    reg = provider_registry("cpu")
    assert "cpu_wan2_2_t2v_14b" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_wan2_2_t2v_14b", LoadSpec.from_dir(snap))
    assert gen.descriptor().modality.name == "VIDEO"
    events = []
    req = dict(prompt="a fox runs", width=256, height=256, steps=3, seed=5, frames=5)
    out = gen.generate(GenerationRequest(**req), events.append)
    assert out.kind == "video" and len(out.video_frames) == 5 and out.fps == 16
    assert all(len(f.pixels) == 256 * 256 * 3 for f in out.video_frames)
    assert [e.current for e in events if hasattr(e, "current")] == [1, 2, 3]
    again = gen.generate(GenerationRequest(**req))
    assert [f.pixels for f in again.video_frames] == [f.pixels for f in out.video_frames]
    other = gen.generate(GenerationRequest(**{**req, "guidance": 1.0}))
    assert [f.pixels for f in other.video_frames] != [f.pixels for f in out.video_frames]
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(**{**req, "frames": 6}))
    cancelled = GenerationRequest(**req)
    cancelled.cancel.cancel()
    from inference_b200.contracts.errors import Canceled
    with pytest.raises(Canceled):
        gen.generate(cancelled)


def test_wan_trainer(tmp_path):
    from inference_b200.contracts.gen_core import LoadSpec, TrainingConfig
    from inference_b200.io.safetensors_io import load_file, save_file
    from inference_b200.media import provider_registry
    from inference_b200.media.train import WAN_TARGETS
    from inference_b200.media.wan import write_synthetic_snapshot
    from inference_b200.testkit.aux_suites import TrainerProfile, trainer_conformance

    snap = write_synthetic_snapshot(tmp_path / "wan")
    ds = tmp_path / "ds"
    ds.mkdir()
    g = torch.Generator().manual_seed(0)
    for i in range(2):
        save_file({"latent": torch.randn(16, 2, 4, 4, generator=g), "txt": torch.randn(7, 64, generator=g)}, ds / f"item{i}.safetensors")
    reg = provider_registry("cpu")
    tr = reg.load_kind("trainer", "cpu_wan_lora_trainer", LoadSpec.from_dir(snap))
    items = tr._items(ds)
    noise = torch.randn(16, 2, 4, 4, generator=torch.Generator().manual_seed(9))
    before = float(tr.loss_on(items[0], 0.5, noise))
    final = tr.train(TrainingConfig(dataset_dir=ds, output_dir=tmp_path / "run", steps=8, learning_rate=5e-3, rank=4, alpha=4.0,
                                    seed=3), lambda p: None)
    ad = load_file(final)
    assert all(k.split(".lora_")[0].endswith(WAN_TARGETS) for k in ad) and len(ad) == 2 * 2 * 8
    tr.model.lora = {k[len("transformer."):-len(".lora_A.weight")]: (ad[k], ad[k.replace("lora_A", "lora_B")], 1.0)
                     for k in ad if k.endswith("lora_A.weight")}
    assert float(tr.loss_on(items[0], 0.5, noise)) < before
    tr.model.lora = None
    trainer_conformance(reg.load_kind("trainer", "cpu_wan_lora_trainer", LoadSpec.from_dir(snap)),
                        TrainerProfile(ds, tmp_path / "out", steps=3, rank=2))


def test_flow_unipc_integrator():
    from inference_b200.media.wan import FlowUniPc, wan_sigmas

    g = torch.Generator().manual_seed(0)
    target, noise = torch.randn(6, generator=g), torch.randn(6, generator=g)
    # a model that always predicts the same clean sample: every consistent integrator must land on it exactly
    sig = wan_sigmas(6, 3.0)
    x, st = noise * sig[0] + target * (1 - sig[0]), FlowUniPc(sig)
    first = None
    for i in range(6):
        v = (x - target) / sig[i]
        nxt = st.step(v, x, i)
        if i == 0:
            first = nxt
            torch.testing.assert_close(first, x + v * (sig[1] - sig[0]))          # the warm-up step is the Euler step
        x = nxt
    torch.testing.assert_close(x, target, atol=1e-5, rtol=1e-5)
    # a curved problem, x0(x, sigma) = tanh(x): the multistep integrator is closer to a fine Euler run than coarse Euler
    def run(n, unipc):
        s = wan_sigmas(n, 3.0)
        z = noise.double() * s[0]
        stp = FlowUniPc(s)
        for i in range(n):
            v = (z - torch.tanh(z)) / s[i]
            z = stp.step(v, z, i) if unipc else z + v * (s[i + 1] - s[i])
        return z
    fine = run(400, False)
    assert (run(10, True) - fine).abs().max() < (run(10, False) - fine).abs().max()


def test_wan_vae_encoder_is_causal_and_streams():
    """Encoding a prefix of the clip gives the prefix of the latents (what the reference's chunked streaming encode
    relies on), the first latent frame depends on frame 0 only, and the frame count law 1 + 4n -> 1 + n holds."""
    from inference_b200.models.vae_qwen import QwenVaeConfig, WanVaeEncoder, random_wan_vae_encoder_weights

    cfg = QwenVaeConfig(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    enc = WanVaeEncoder(cfg, random_wan_vae_encoder_weights(cfg, seed=1, std=0.2))
    v = torch.randn(1, 3, 9, 16, 24)
    z = enc.encode(v)
    assert z.shape == (1, 16, 3, 2, 3)
    assert torch.allclose(enc.encode(v[:, :, :5]), z[:, :, :2], atol=1e-5)
    assert torch.allclose(enc.encode(v[:, :, :1]), z[:, :, :1], atol=1e-5)
    v2 = v.clone()
    v2[:, :, 1:] += 1.0
    z2 = enc.encode(v2)
    assert torch.equal(z2[:, :, 0], z[:, :, 0]) and not torch.allclose(z2[:, :, 1], z[:, :, 1], atol=1e-4)
    with pytest.raises(ValueError):
        enc.encode(v[:, :, :6])


def test_wan_i2v_provider(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media import provider_registry
    from inference_b200.media.wan import I2V_14B, preprocess_i2v_image, write_synthetic_snapshot

    assert (I2V_14B.boundary, I2V_14B.shift, I2V_14B.guidance_high, I2V_14B.guidance_low) == (0.9, 5.0, 3.5, 3.5)
    # cover-fit: a 4x2 image onto 2x2 keeps the centre columns; values map to [-1, 1]
    img = Image(4, 2, bytes([0, 0, 0, 255, 255, 255, 255, 255, 255, 0, 0, 0] * 2))
    t = preprocess_i2v_image(img, 2, 2)
    assert t.shape == (1, 3, 1, 2, 2) and torch.allclose(t, torch.ones_like(t))
    snap = write_synthetic_snapshot(tmp_path / "wan_i2v", i2v=True)
    reg = provider_registry("cpu")
    assert {"cpu_wan2_2_t2v_14b", "cpu_wan2_2_i2v_14b"} <= set(reg.ids()) and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_wan2_2_i2v_14b", LoadSpec.from_dir(snap))
    assert gen.descriptor().capabilities.accepts(ConditioningKind.REFERENCE)
    g = torch.Generator().manual_seed(0)
    ref = Image(48, 32, torch.randint(0, 255, (32 * 48 * 3,), generator=g, dtype=torch.uint8).numpy().tobytes())
    req = dict(prompt="the fox turns its head", width=256, height=256, steps=2, seed=5, frames=5)
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(**req))                               # no reference image
    cond = [Conditioning(kind=ConditioningKind.REFERENCE, image=ref)]
    out = gen.generate(GenerationRequest(**req, conditioning=cond))
    assert len(out.video_frames) == 5 and out.fps == 16
    ref2 = Image(48, 32, bytes(32 * 48 * 3))
    other = gen.generate(GenerationRequest(**req, conditioning=[Conditioning(kind=ConditioningKind.REFERENCE, image=ref2)]))
    assert [f.pixels for f in other.video_frames] != [f.pixels for f in out.video_frames]
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(**{**req, "width": 1280, "height": 1280}, conditioning=cond))
