"""Stable Video Diffusion: schedule and preconditioning values stated by the reference's tests, the UNet's blending and
frame-batching structure (a temporal branch that is switched off leaves frames independent; switched on it couples
them), the autoencoder's chunk invariance, and provider conformance with a Reference image."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.models import unet_svd as S

UCFG = S.SvdUnetConfig(block_out_channels=(8, 16), num_attention_heads=(2, 2), cross_attention_dim=12,
                       addition_time_embed_dim=4, projection_class_embeddings_input_dim=12, groups=4)
VCFG = S.SvdVaeConfig(block_out_channels=(8, 8, 8, 16), layers_per_block=1, groups=4)


def test_karras_table_and_edm_preconditioning():
    from inference_b200.contracts.gen_core.sampling import EdmModelSampling

    s = S.karras_sigmas(25)
    assert len(s) == 26 and abs(s[0] - 700.0) < 1e-1 and abs(s[24] - 0.002) < 1e-4 and s[25] == 0.0
    assert all(a > b for a, b in zip(s, s[1:]))
    ms = EdmModelSampling(0.002, 700.0)
    assert abs(ms.timestep(700.0) - 0.25 * math.log(700.0)) < 1e-6
    kx, ko = ms.denoised_coeffs(3.0)
    assert abs(kx - 1 / 10.0) < 1e-9 and abs(ko + 3.0 / math.sqrt(10.0)) < 1e-9 and abs(ms.input_scale(3.0) - 1 / math.sqrt(10.0)) < 1e-9


def test_unet_structure_and_temporal_coupling():
    w = S.random_svd_unet_weights(UCFG, seed=1)
    x = torch.randn(1, 3, 8, 8, 8)
    emb, ids = torch.randn(1, 1, 12), torch.tensor([[6.0, 127.0, 0.02]])
    out = S.SvdUnet(UCFG, w).forward(x, 1.2, emb, ids)
    assert out.shape == (1, 3, 4, 8, 8) and torch.isfinite(out).all()
    # mix factors at +large: sigmoid -> 1, so every block keeps its spatial branch only and frames do not interact
    w_sp = {k: (torch.full_like(v, 30.0) if k.endswith("mix_factor") else v) for k, v in w.items()}
    net = S.SvdUnet(UCFG, w_sp)
    full = net.forward(x, 1.2, emb, ids)
    single = torch.cat([net.forward(x[:, f:f + 1], 1.2, emb, ids) for f in range(3)], 1)
    assert torch.allclose(full, single, atol=1e-4), (full - single).abs().max()
    x2 = x.clone()
    x2[:, 2] += 1.0
    a, b = S.SvdUnet(UCFG, w).forward(x, 1.2, emb, ids), S.SvdUnet(UCFG, w).forward(x2, 1.2, emb, ids)
    assert not torch.allclose(a[:, 0], b[:, 0], atol=1e-5)           # with the temporal branch on, frame 2 reaches frame 0
    # one spatio-temporal block against its definition
    p, frames = "mid_block.resnets.0", 3
    h = torch.randn(3, 16, 4, 4)
    temb = torch.randn(3, 32)
    net = S.SvdUnet(UCFG, w)
    s = net.spatial_res(h, p + ".spatial_res_block", 1e-5, temb)
    s5 = s.reshape(1, 3, 16, 4, 4).permute(0, 2, 1, 3, 4)
    t = p + ".temporal_res_block"
    y = F.conv3d(F.silu(F.group_norm(s5, 4, w[t + ".norm1.weight"], w[t + ".norm1.bias"], 1e-5)), w[t + ".conv1.weight"], w[t + ".conv1.bias"], padding=(1, 0, 0))
    y = y + F.linear(F.silu(temb), w[t + ".time_emb_proj.weight"], w[t + ".time_emb_proj.bias"]).t()[None, :, :, None, None]
    y = s5 + F.conv3d(F.silu(F.group_norm(y, 4, w[t + ".norm2.weight"], w[t + ".norm2.bias"], 1e-5)), w[t + ".conv2.weight"], w[t + ".conv2.bias"], padding=(1, 0, 0))
    al = torch.sigmoid(w[p + ".time_mixer.mix_factor"])
    want = (s5 * al + y * (1 - al)).permute(0, 2, 1, 3, 4).reshape(3, 16, 4, 4)
    assert torch.allclose(net.st_res(h, p, 1e-5, frames, temb), want, atol=1e-5)


def test_vae_roundtrip_shapes_and_blend_direction():
    w = S.random_svd_vae_weights(VCFG, seed=2)
    vae = S.SvdVae(VCFG, w)
    lat = vae.encode_mode(torch.randn(1, 3, 32, 48))
    assert lat.shape == (1, 4, 4, 6)
    z = torch.randn(4, 4, 4, 6)
    video = vae.decode(z, 4)
    assert video.shape == (4, 3, 32, 48)
    # decoder blend is (1 - alpha) * spatial + alpha * temporal: with alpha -> 0 frames decode independently up to the
    # final 3-tap temporal convolution
    w0 = {k: (torch.full_like(v, -30.0) if k.endswith("mix_factor") else v) for k, v in w.items()}
    w0["decoder.time_conv_out.weight"] = torch.zeros_like(w0["decoder.time_conv_out.weight"])
    w0["decoder.time_conv_out.weight"][:, :, 1, 0, 0] = torch.eye(3)
    v0 = S.SvdVae(VCFG, w0)
    assert torch.allclose(v0.decode(z, 4), torch.cat([v0.decode(z[i:i + 1], 1) for i in range(4)]), atol=1e-4)


def test_svd_provider_conforms(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.media import provider_registry
    from inference_b200.media.svd import write_synthetic_snapshot
    from inference_b200.testkit import generator as kit

    snap = write_synthetic_snapshot(tmp_path / "svd")
    reg = provider_registry("cpu")
    assert "cpu_svd_xt" in reg.ids() and reg.descriptor_conformance_errors() == []
    gen = reg.load("cpu_svd_xt", LoadSpec.from_dir(snap))
    g = torch.Generator().manual_seed(0)
    ref = Image(40, 30, torch.randint(0, 255, (30 * 40 * 3,), generator=g, dtype=torch.uint8).numpy().tobytes())
    cond = (Conditioning(kind=ConditioningKind.REFERENCE, image=ref),)
    kit.conformance(gen, kit.Profile(prompt="", width=64, height=64, steps=2, cancel_steps=4, conditioning=cond))
    req = dict(prompt="", width=64, height=64, steps=2, seed=4, frames=3, conditioning=list(cond))
    out = gen.generate(GenerationRequest(**req))
    assert len(out.video_frames) == 3 and out.fps == 7 and len(out.video_frames[0].pixels) == 64 * 64 * 3
    chunked = gen.generate(GenerationRequest(**req, decode_chunk_size=3, motion_bucket_id=30.0))
    assert kit.output_bytes(chunked) != kit.output_bytes(out)
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(prompt="", width=64, height=64, steps=2))
    with pytest.raises(InferenceError):
        gen.generate(GenerationRequest(**{**req, "frames": 65}))
