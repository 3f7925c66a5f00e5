"""FLUX-style DiT on sm_100a kernels vs the fp32 oracle (small head_dim-128 config), plus the media kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_media_kernels():
    from inference_b200 import ops

    x = torch.randn(1000, 64, device="cuda").bfloat16()
    y = torch.randn(1000, 64, device="cuda").bfloat16()
    z = ops.axpy(1.0, x, -0.3, y)
    assert torch.allclose(z.float(), x.float() - 0.3 * y.float(), atol=2e-2)
    zf = ops.axpy(0.5, x.float(), 2.0, y.float())
    assert torch.allclose(zf, 0.5 * x.float() + 2.0 * y.float(), atol=1e-5)
    a = torch.randn(2, 24, 20, 64, device="cuda").bfloat16()
    g = (torch.rand(64, device="cuda") + 0.5).bfloat16()
    b = (torch.randn(64, device="cuda") * 0.1).bfloat16()
    for silu in (False, True):
        out = ops.groupnorm_nhwc(a, g, b, groups=8, eps=1e-6, silu=silu)
        ref = torch.nn.functional.group_norm(a.float().permute(0, 3, 1, 2), 8, g.float(), b.float(), 1e-6)
        if silu:
            ref = torch.nn.functional.silu(ref)
        assert torch.allclose(out.float(), ref.permute(0, 2, 3, 1), atol=4e-2, rtol=2e-2)
    for C, G in ((128, 32), (64, 32), (32, 32)):      # groups narrower than one 16-byte vector
        a2 = torch.randn(2, 9, 7, C, device="cuda").bfloat16()
        g2 = (torch.rand(C, device="cuda") + 0.5).bfloat16()
        b2 = (torch.randn(C, device="cuda") * 0.1).bfloat16()
        out = ops.groupnorm_nhwc(a2, g2, b2, groups=G, eps=1e-6, silu=True)
        ref = torch.nn.functional.silu(torch.nn.functional.group_norm(a2.float().permute(0, 3, 1, 2), G, g2.float(),
                                                                      b2.float(), 1e-6))
        assert torch.allclose(out.float(), ref.permute(0, 2, 3, 1), atol=4e-2, rtol=2e-2)
    # wide groups on the row-coalesced statistics kernel, small and large maps, several samples; and a channel count
    # whose vector columns do not divide the CTA (the one-vector-per-thread kernels)
    for N, H, W, C, G in ((2, 64, 64, 256, 32), (1, 16, 16, 512, 32), (3, 5, 7, 512, 32), (1, 9, 11, 192, 8)):
        a2 = (torch.randn(N, H, W, C, device="cuda") * 2 + 0.5).bfloat16()
        g2 = (torch.rand(C, device="cuda") + 0.5).bfloat16()
        b2 = (torch.randn(C, device="cuda") * 0.1).bfloat16()
        out = ops.groupnorm_nhwc(a2, g2, b2, groups=G, eps=1e-6, silu=True)
        ref = torch.nn.functional.silu(torch.nn.functional.group_norm(a2.float().permute(0, 3, 1, 2), G, g2.float(),
                                                                      b2.float(), 1e-6))
        assert torch.allclose(out.float(), ref.permute(0, 2, 3, 1), atol=4e-2, rtol=2e-2), (N, H, W, C, G)
    a3 = torch.randn(1, 5, 6, 16, device="cuda").bfloat16()
    cols = ops.im2col3x3_nhwc(a3)
    ref = torch.nn.functional.unfold(a3.float().permute(0, 3, 1, 2), 3, padding=1)      # [1, C*9, L], (c, kh, kw)
    ref = ref.view(1, 16, 9, 30).permute(0, 3, 2, 1).reshape(30, 144)
    assert torch.equal(cols.float(), ref)
    up = ops.upsample2x_nhwc(a)
    ref = torch.nn.functional.interpolate(a.float().permute(0, 3, 1, 2), scale_factor=2, mode="nearest")
    assert torch.equal(up.float(), ref.permute(0, 2, 3, 1))
    s = torch.randn(37, 1000, device="cuda")
    p = ops.softmax_rows(s, 0.5)
    assert torch.allclose(p.float(), torch.softmax(s * 0.5, -1), atol=2e-3)
    img = (torch.rand(1, 16, 16, 8, device="cuda") * 2.4 - 1.2).bfloat16()
    u8 = ops.rgb8_nhwc(img)
    ref = torch.round((img[..., :3].float().clamp(-1, 1) + 1) * 127.5).to(torch.uint8)
    assert torch.equal(u8, ref)


def test_rope_in_place_updates_k_without_cache():
    from inference_b200 import ops

    T, H, D = 6, 2, 128
    qkv = torch.randn(T, 3 * H * D, device="cuda").bfloat16()
    before = qkv.clone()
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    ang = torch.arange(T, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(0, D, 2) / D))[None]
    cos, sin = ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous()
    ops.rope_kv_write(qkv, pos, None, cos, sin, None, None, H, H, D, interleaved=True)
    k_before = before[:, H * D:2 * H * D].float().view(T, H, D)
    x0, x1 = k_before[..., 0::2], k_before[..., 1::2]
    ref = torch.stack((x0 * cos[:, None] - x1 * sin[:, None], x1 * cos[:, None] + x0 * sin[:, None]), -1).flatten(-2)
    got = qkv[:, H * D:2 * H * D].float().view(T, H, D)
    assert torch.allclose(got, ref, atol=3e-2)
    assert torch.equal(qkv[:, 2 * H * D:], before[:, 2 * H * D:])


@pytest.mark.parametrize("batch", [1, 2])
def test_flux_dit_matches_oracle(batch):
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT, make_ids, random_flux_weights

    cfg = FluxConfig(in_channels=64, vec_in_dim=64, context_in_dim=128, hidden_size=256, num_heads=2, depth=2,
                     depth_single=2)
    w = {k: v.bfloat16().float() for k, v in random_flux_weights(cfg, seed=0, std=0.05).items()}
    oracle = OracleFluxDiT(cfg, w, device="cuda")
    model = FluxDiTGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
    g = torch.Generator(device="cuda").manual_seed(3)
    hh, ww, St = 6, 5, 19
    img = torch.randn(batch, hh * ww, 64, device="cuda", generator=g).bfloat16()
    txt = torch.randn(batch, St, 128, device="cuda", generator=g).bfloat16()
    y = torch.randn(batch, 64, device="cuda", generator=g).bfloat16()
    t = torch.full((batch,), 0.7, device="cuda")
    gd = torch.full((batch,), 3.5, device="cuda")
    txt_ids, img_ids = make_ids(hh, ww, St, "cuda")
    ref = oracle.forward(img.float(), img_ids, txt.float(), txt_ids, t, y.float(), gd)
    out = model.forward(img, img_ids, txt, txt_ids, t, y, gd)
    err = (out.float() - ref).abs().max().item()
    assert err < 0.06 * max(1.0, ref.abs().max().item()), err
    # graph replay: first call captures, second replays with new inputs
    for scale_in in (1.0, 0.5):
        img2 = (img.float() * scale_in).bfloat16()
        eager = model.forward(img2, img_ids, txt, txt_ids, t, y, gd).clone()
        replay = model.forward_graphed(img2, img_ids, txt, txt_ids, t, y, gd)
        assert torch.equal(eager, replay)


def test_flux_dit_image_stream_hooks_match_oracle():
    """The identity-adapter seam: perceiver cross-attention residuals added to the image stream after double / single
    blocks give the same velocity on the device model (eager and through forward_graphed) as on the fp32 oracle."""
    from inference_b200.media.pulid import IdFormerConfig, PulidCa, random_pulid_weights
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT, make_ids, random_flux_weights

    cfg = FluxConfig(in_channels=64, vec_in_dim=64, context_in_dim=128, hidden_size=256, num_heads=2, depth=2,
                     depth_single=2)
    w = {k: v.bfloat16().float() for k, v in random_flux_weights(cfg, seed=0, std=0.05).items()}
    oracle = OracleFluxDiT(cfg, w, device="cuda")
    model = FluxDiTGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
    pw = random_pulid_weights(IdFormerConfig(dim=16, depth=5, heads=2, dim_head=8, output_dim=24), 256, 2, 3)
    pw["swb_ca_config"] = torch.tensor([2, 8])
    g = torch.Generator(device="cuda").manual_seed(5)
    emb = torch.randn(1, 4, 24, device="cuda", generator=g)
    hh, ww, St = 6, 5, 19
    img = torch.randn(1, hh * ww, 64, device="cuda", generator=g).bfloat16()
    txt = torch.randn(1, St, 128, device="cuda", generator=g).bfloat16()
    y = torch.randn(1, 64, device="cuda", generator=g).bfloat16()
    t, gd = torch.full((1,), 0.7, device="cuda"), torch.full((1,), 3.5, device="cuda")
    txt_ids, img_ids = make_ids(hh, ww, St, "cuda")
    plain = model.forward(img, img_ids, txt, txt_ids, t, y, gd).float()
    oracle.injector = model.injector = PulidCa(pw, emb, 1.0, cfg.depth, cfg.depth_single, "cuda")
    ref = oracle.forward(img.float(), img_ids, txt.float(), txt_ids, t, y.float(), gd)
    out = model.forward(img, img_ids, txt, txt_ids, t, y, gd).float()
    assert (out - ref).abs().max().item() < 0.06 * max(1.0, ref.abs().max().item())
    assert (out - plain).abs().max().item() > 1e-2
    assert torch.equal(model.forward_graphed(img, img_ids, txt, txt_ids, t, y, gd).float(), out)
    model.injector = None
    assert torch.equal(model.forward(img, img_ids, txt, txt_ids, t, y, gd).float(), plain)


@pytest.mark.parametrize("shape", [(1, 16, 16, 64, 128), (2, 32, 32, 128, 64), (1, 64, 64, 256, 256), (1, 128, 128, 128, 128),
                                   (1, 8, 256, 64, 8), (3, 4, 32, 64, 16)])
def test_implicit_conv3x3_matches_conv2d(shape, monkeypatch):
    """3x3 convolution as an implicit GEMM (TMA-shifted taps, zero fill as padding) against F.conv2d in fp32: tiles
    that are part of a row, whole rows and stacks of rows; bias, activation and residual epilogues; several images
    per batch (a tile never straddles two images); and agreement with the patch-gather path."""
    import torch.nn.functional as F

    from inference_b200 import ops

    N, H, W, C, Co = shape
    g = torch.Generator(device="cuda").manual_seed(H * W + C)
    x = torch.randn(N, H, W, C, device="cuda", generator=g).bfloat16()
    w4 = (torch.randn(Co, C, 3, 3, device="cuda", generator=g) / (9 * C) ** 0.5).bfloat16()
    b = torch.randn(Co, device="cuda", generator=g).bfloat16()
    r = torch.randn(N, H, W, Co, device="cuda", generator=g).bfloat16()
    wk = w4.permute(0, 2, 3, 1).reshape(Co, 9 * C).contiguous()
    assert ops.conv3x3_supported(x)
    ref = F.conv2d(x.float().permute(0, 3, 1, 2), w4.float(), b.float(), padding=1).permute(0, 2, 3, 1)
    got = ops.conv3x3_nhwc(x, wk, b)
    assert got.shape == (N, H, W, Co)
    assert (got.float() - ref).abs().max().item() < 0.03 * max(1.0, ref.abs().max().item())
    got = ops.conv3x3_nhwc(x, wk, b, residual=r, act="silu")
    want = F.silu(ref) + r.float()
    assert (got.float() - want).abs().max().item() < 0.03 * max(1.0, want.abs().max().item())
    monkeypatch.setenv("SWB_CONV3X3", "im2col")
    old = ops.conv3x3_nhwc(x, wk, b)
    assert (old.float() - ops.conv3x3_nhwc(x, wk, b).float()).abs().max().item() == 0.0
    monkeypatch.setenv("SWB_CONV3X3", "implicit")
    assert (old.float() - ops.conv3x3_nhwc(x, wk, b).float()).abs().max().item() < 0.02 * max(1.0, ref.abs().max().item())
    narrow = torch.randn(1, 16, 16, 16, device="cuda", generator=g).bfloat16()          # 16 channels: the gather path
    assert not ops.conv3x3_supported(narrow)
    wn = (torch.randn(32, 16, 3, 3, device="cuda", generator=g) / 12).bfloat16()
    out = ops.conv3x3_nhwc(narrow, wn.permute(0, 2, 3, 1).reshape(32, 144).contiguous())
    refn = F.conv2d(narrow.float().permute(0, 3, 1, 2), wn.float(), padding=1).permute(0, 2, 3, 1)
    assert (out.float() - refn).abs().max().item() < 0.03 * max(1.0, refn.abs().max().item())


def test_vae_decoder_matches_oracle():
    from inference_b200.models.vae import OracleVaeDecoder, VaeConfig, VaeDecoderGpu, random_vae_weights

    cfg = VaeConfig(ch=64, ch_mult=(1, 2), num_res_blocks=1)
    w = {k: v.bfloat16().float() for k, v in random_vae_weights(cfg, seed=0).items()}
    oracle = OracleVaeDecoder(cfg, w, device="cuda")
    gpu = VaeDecoderGpu(cfg, torch.device("cuda")).load_state_dict(w)
    z = torch.randn(1, 16, 12, 10, device="cuda") * 0.5
    ref = oracle.decode(z)                                  # [1, 3, 24, 20]
    out = gpu.decode(z)[..., :3].permute(0, 3, 1, 2).float()
    assert out.shape == ref.shape
    err = (out - ref).abs().max().item()
    assert err < 0.06 * max(1.0, ref.abs().max().item()), err
    u8 = gpu.decode_rgb8(z)
    assert u8.shape == (1, 24, 20, 3) and u8.dtype == torch.uint8


def test_chroma_dit_matches_oracle():
    from inference_b200.models.dit_chroma import ChromaConfig, ChromaDiTGpu, OracleChromaDiT, random_chroma_weights
    from inference_b200.models.dit_flux import make_ids

    cfg = ChromaConfig(in_channels=64, num_layers=2, num_single_layers=2, attention_head_dim=128, num_attention_heads=2,
                       joint_attention_dim=128, approximator_num_channels=64, approximator_hidden_dim=128,
                       approximator_layers=2)
    w = {k: v.bfloat16().float() for k, v in random_chroma_weights(cfg, seed=0, std=0.05).items()}
    oracle = OracleChromaDiT(cfg, w, device="cuda")
    model = ChromaDiTGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
    g = torch.Generator(device="cuda").manual_seed(3)
    hh, ww, St = 6, 5, 19
    img = torch.randn(1, hh * ww, 64, device="cuda", generator=g).bfloat16()
    txt = torch.randn(1, St, 128, device="cuda", generator=g).bfloat16()
    t = torch.full((1,), 0.7, device="cuda")
    txt_ids, img_ids = make_ids(hh, ww, St, "cuda")
    ref = oracle.forward(img.float(), img_ids, txt.float(), txt_ids, t, None, None)
    out = model.forward(img, img_ids, txt, txt_ids, t, None, None)
    err = (out.float() - ref).abs().max().item()
    assert err < 0.06 * max(1.0, ref.abs().max().item()), err
    eager = out.clone()
    for _ in range(2):                                         # capture, then replay
        assert torch.equal(eager, model.forward_graphed(img, img_ids, txt, txt_ids, t, None, None))


def _reference_conditioning():
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image

    g = torch.Generator().manual_seed(0)
    px = torch.randint(0, 255, (30 * 40 * 3,), generator=g, dtype=torch.uint8).numpy().tobytes()
    return [Conditioning(kind=ConditioningKind.REFERENCE, image=Image(40, 30, px))]


# families built on media/family.py: module name -> (model id, request extras)
FAMILY_TABLE = {
    "svd": ("svd_xt", {"prompt": "", "frames": 3, "width": 64, "height": 64, "conditioning": _reference_conditioning()}),
    "krea": ("krea_2_raw", {"guidance": 2.0, "negative_prompt": "blurry"}),
    "flux2": ("flux2_klein_9b", {"guidance": 2.0, "negative_prompt": "blurry"}),
    "sana": ("sana_1600m", {"guidance": 2.0, "negative_prompt": "blurry"}),
    "ideogram": ("ideogram_4", {"guidance": 2.0}),
    "anima": ("anima_base", {"guidance": 2.0, "negative_prompt": "blurry", "width": 512, "height": 512}),
    "mochi": ("mochi_1", {"guidance": 2.0, "negative_prompt": "blurry", "frames": 7}),
    "boogu": ("boogu_image", {"guidance": 2.0}),
    "sensenova": ("sensenova_u1_8b", {"guidance": 2.0}),
    "wan_ti2v": ("wan2_2_ti2v_5b", {"guidance": 2.0, "sampler": "euler", "frames": 5, "width": 480, "height": 512}),
    "wan_vace": ("wan_vace", {"guidance": 2.0, "sampler": "euler", "conditioning": "vace"}),
    "scail2": ("scail2_14b", {"guidance": 2.0, "sampler": "euler", "width": 64, "height": 64, "conditioning": "scail2"}),
    "bernini": ("bernini_renderer", {"guidance": 2.0, "frames": 5, "width": 64, "height": 64, "sampler": "euler"}),
}


@pytest.mark.parametrize("family", ["flux", "chroma", "z_image", "sd3", "qwen_image", "sdxl", "kolors", *FAMILY_TABLE])
def test_generator_providers_on_device_track_the_oracle_backend(tmp_path, family):
    """The sm_100a provider and the fp32 oracle provider render the same snapshot, seed and request."""
    import numpy as np

    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry

    if family in FAMILY_TABLE:
        import importlib

        write_synthetic_snapshot = importlib.import_module(f"inference_b200.media.{family}").write_synthetic_snapshot
        mid, extra = FAMILY_TABLE[family]
    elif family == "flux":
        from inference_b200.media.flux import write_synthetic_snapshot
        mid, extra = "flux1_dev", {}
    elif family == "chroma":
        from inference_b200.media.chroma import write_synthetic_snapshot
        mid, extra = "chroma1_hd", {"true_cfg": 2.0, "negative_prompt": "blurry"}
    elif family == "sdxl":
        from inference_b200.media.sdxl import write_synthetic_snapshot
        mid, extra = "sdxl", {"guidance": 2.0, "negative_prompt": "blurry"}
    elif family == "kolors":
        from inference_b200.media.kolors import write_synthetic_snapshot as ko

        write_synthetic_snapshot = lambda root: ko(root, text="chatglm")      # noqa: E731
        mid, extra = "kolors", {"guidance": 2.0, "negative_prompt": "blurry"}
    elif family == "qwen_image":
        from inference_b200.media.qwen_image import write_synthetic_snapshot as qi

        write_synthetic_snapshot = lambda root: qi(root, text="qwen_vl", te_head_dim=128)      # noqa: E731
        mid, extra = "qwen_image", {"true_cfg": 2.0, "negative_prompt": "blurry"}
    elif family == "sd3":
        from inference_b200.media.sd3 import write_synthetic_snapshot as s3

        write_synthetic_snapshot = lambda root: s3(root, dual=True)      # noqa: E731
        mid, extra = "sd3_5_medium", {"guidance": 2.0, "negative_prompt": "blurry"}
    else:
        from inference_b200.media.z_image import write_synthetic_snapshot as zi

        write_synthetic_snapshot = lambda root: zi(root, text="qwen3", te_head_dim=128)      # noqa: E731
        mid, extra = "z_image", {"guidance": 2.0, "negative_prompt": "blurry"}
    snap = write_synthetic_snapshot(tmp_path / family)
    req = {**dict(prompt="a lighthouse at dusk", width=256, height=256, steps=2, seed=11), **extra}
    if req.get("conditioning") == "vace":
        from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
        from inference_b200.contracts.gen_core.media import Image

        fr = [Image(64, 64, bytes((i * k) % 256 for i in range(64 * 64 * 3))) for k in (3, 5, 7, 11, 13)]
        mk = [Image(64, 64, bytes([255 * (j >= 2)]) * (64 * 64 * 3)) for j in range(5)]
        req["conditioning"] = [Conditioning(ConditioningKind.CONTROL_CLIP, frames=fr, mask_frames=mk)]
    if req.get("conditioning") == "scail2":
        from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
        from inference_b200.contracts.gen_core.media import Image

        im = lambda k: Image(64, 64, bytes((i * k) % 256 for i in range(64 * 64 * 3)))      # noqa: E731
        req["conditioning"] = [Conditioning(ConditioningKind.REFERENCE, image=im(17)), Conditioning(ConditioningKind.MASK, image=im(19)),
                               Conditioning(ConditioningKind.CONTROL_CLIP, frames=[im(k) for k in (3, 5, 7, 11, 13)],
                                            mask_frames=[im(k + 1) for k in (3, 5, 7, 11, 13)])]
    imgs = {}
    for backend, prefix in (("b200", ""), ("cpu", "cpu_")):
        g = provider_registry(backend).load(prefix + mid, LoadSpec.from_dir(snap))
        out = g.generate(GenerationRequest(**req))
        im = (out.images or out.video_frames)[-1]
        assert (im.width, im.height) == (req["width"], req["height"])
        imgs[backend] = np.frombuffer(im.pixels, dtype=np.uint8).astype(np.float32)
    diff = float(np.abs(imgs["b200"] - imgs["cpu"]).mean())
    assert diff < 8.0, diff


def test_z_image_dit_matches_oracle():
    from inference_b200.models.dit_zimage import OracleZImageDiT, ZImageConfig, ZImageDiTGpu, random_zimage_weights

    cfg = ZImageConfig(dim=384, n_layers=2, n_refiner_layers=1, n_heads=3, cap_feat_dim=64)
    w = {k: v.bfloat16().float() for k, v in random_zimage_weights(cfg, seed=0, std=0.05).items()}
    oracle = OracleZImageDiT(cfg, w, device="cuda")
    model = ZImageDiTGpu(cfg, torch.device("cuda")).load_state_dict(w)
    g = torch.Generator(device="cuda").manual_seed(3)
    z = torch.randn(1, 16, 12, 10, device="cuda", generator=g).bfloat16()
    cap = torch.randn(1, 37, 64, device="cuda", generator=g).bfloat16()
    t = torch.full((1,), 0.3, device="cuda")
    ref = oracle.forward(z.float(), t, cap.float())
    tokens = model.refine_caption(cap)
    ref_tokens = oracle.refine_caption(cap.float())[0]
    assert (tokens.float() - ref_tokens).abs().max().item() < 0.06 * max(1.0, ref_tokens.abs().max().item())
    out = model.forward(z, t, tokens)
    err = (out.float() - ref).abs().max().item()
    assert out.shape == ref.shape and err < 0.06 * max(1.0, ref.abs().max().item()), err
    eager = out.clone()
    for _ in range(2):                                         # capture, then replay
        assert torch.equal(eager, model.forward_graphed(z, t, tokens))


def test_causal_lm_prompt_encoder_matches_oracle():
    from inference_b200.models.config import ModelConfig
    from inference_b200.models.oracle import OracleLlama, random_llama_weights
    from inference_b200.models.text_encoders import CausalLmTextEncoder

    cfg = ModelConfig.from_json({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 256,
                                 "intermediate_size": 512, "num_hidden_layers": 3, "num_attention_heads": 4,
                                 "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 300, "rms_norm_eps": 1e-6,
                                 "rope_theta": 1000000.0, "tie_word_embeddings": True})
    w = {k: v.bfloat16().float() for k, v in random_llama_weights(cfg, 1, std=0.05).items()}
    enc = CausalLmTextEncoder(cfg, w, "cuda")
    assert enc.native
    ids = [5, 17, 200, 3, 99, 42, 7, 250, 11]
    out = enc.encode(ids)
    ref = OracleLlama(cfg, w, device="cuda").hidden_states(torch.tensor([ids], device="cuda"), None, num_layers=2)
    assert out.shape == ref.shape
    assert (out.float() - ref).abs().max().item() < 0.05 * max(1.0, ref.abs().max().item())


def test_qwen_image_dit_matches_oracle():
    from inference_b200.models.dit_qwen_image import (OracleQwenImageDiT, QwenImageConfig, QwenImageDiTGpu, position_ids,
                                                      random_qwen_image_weights)

    cfg = QwenImageConfig(num_layers=2, num_attention_heads=2, joint_attention_dim=128)
    w = {k: v.bfloat16().float() for k, v in random_qwen_image_weights(cfg, seed=0, std=0.05).items()}
    oracle = OracleQwenImageDiT(cfg, w, device="cuda")
    model = QwenImageDiTGpu(cfg, device=torch.device("cuda")).load_state_dict(w)
    g = torch.Generator(device="cuda").manual_seed(3)
    hh, ww, St = 6, 5, 19
    img = torch.randn(1, hh * ww, 64, device="cuda", generator=g).bfloat16()
    txt = torch.randn(1, St, 128, device="cuda", generator=g).bfloat16()
    t = torch.full((1,), 0.7, device="cuda")
    txt_ids, img_ids = position_ids(hh, ww, St, "cuda")
    ref = oracle.forward(img.float(), img_ids, oracle.prepare_text(txt.float()), txt_ids, t, None, None)
    ptxt = model.prepare_text(txt)
    out = model.forward(img, img_ids, ptxt, txt_ids, t, None, None)
    err = (out.float() - ref).abs().max().item()
    assert err < 0.06 * max(1.0, ref.abs().max().item()), err
    eager = out.clone()
    for _ in range(2):
        assert torch.equal(eager, model.forward_graphed(img, img_ids, ptxt, txt_ids, t, None, None))


def test_wan_dit_on_device_matches_fp32_and_provider_renders_frames(tmp_path):
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.media import provider_registry
    from inference_b200.media.wan import write_synthetic_snapshot
    from inference_b200.models.dit_wan import WanConfig, WanDiT, random_wan_weights

    cfg = WanConfig(num_attention_heads=2, attention_head_dim=128, num_layers=2, ffn_dim=256, text_dim=64)
    w = {k: v.bfloat16().float() for k, v in random_wan_weights(cfg, seed=0, std=0.05).items()}
    ref_model = WanDiT(cfg, w, torch.float32, "cuda")
    model = WanDiT(cfg, w, torch.bfloat16, "cuda")
    g = torch.Generator(device="cuda").manual_seed(3)
    z = torch.randn(1, 16, 3, 8, 12, device="cuda", generator=g).bfloat16()
    ctx = torch.randn(1, 21, 64, device="cuda", generator=g).bfloat16()
    t = torch.full((1,), 600.0, device="cuda")
    ref = ref_model.forward(z.float(), t, ctx.float())
    out = model.forward(z, t, ctx)
    err = (out.float() - ref).abs().max().item()
    assert out.shape == ref.shape and err < 0.06 * max(1.0, ref.abs().max().item()), err
    snap = write_synthetic_snapshot(tmp_path / "wan")
    req = dict(prompt="a fox runs", width=256, height=256, steps=2, seed=5, frames=5)
    import numpy as np

    vids = {}
    for backend, prefix in (("b200", ""), ("cpu", "cpu_")):
        gen = provider_registry(backend).load(prefix + "wan2_2_t2v_14b", LoadSpec.from_dir(snap))
        o = gen.generate(GenerationRequest(**req))
        assert len(o.video_frames) == 5
        vids[backend] = np.frombuffer(b"".join(f.pixels for f in o.video_frames), dtype=np.uint8).astype(np.float32)
    assert float(np.abs(vids["b200"] - vids["cpu"]).mean()) < 8.0


@pytest.mark.parametrize("D,Sq,Skv,B", [(64, 300, 300, 2), (64, 1024, 77, 2), (72, 96, 96, 1), (128, 130, 50, 1)])
def test_padded_dense_attention_serves_narrow_heads(D, Sq, Skv, B):
    from inference_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(D + Sq)
    q = torch.randn(B, Sq, 5, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, Skv, 5, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, Skv, 5, D, device="cuda", generator=g).bfloat16()
    out = ops.dense_attention_padded(q, k, v, scale=D ** -0.5)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float().transpose(1, 2), k.float().transpose(1, 2),
                                                           v.float().transpose(1, 2)).transpose(1, 2).reshape(B, Sq, 5 * D)
    assert out.shape == ref.shape
    assert (out.float() - ref).abs().max().item() < 0.03


def test_flux_control_branch_on_device_tracks_the_oracle():
    """The ControlNet branch on the sm_100a model class (fused checkpoint layout, tcgen05 GEMM / attention) against the
    fp32 oracle class carrying the same converted weights, and the controlled base forward against its fp32 twin."""
    from inference_b200.media import flux_control as C
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT, make_ids, random_flux_weights

    base_cfg = FluxConfig.tiny()
    sd = C.random_control_weights(base_cfg, layers=2, seed=1, std=0.05)
    g = torch.Generator().manual_seed(0)
    ht, wt, St = 8, 8, 16
    img, cond = torch.randn(1, ht * wt, base_cfg.in_channels, generator=g), torch.randn(1, ht * wt, base_cfg.in_channels, generator=g)
    txt, y = torch.randn(1, St, base_cfg.context_in_dim, generator=g), torch.randn(1, base_cfg.vec_in_dim, generator=g)
    txt_ids, img_ids = make_ids(ht, wt, St)
    t, gd = torch.tensor([0.7]), torch.tensor([3.5])
    ref_branch = C.FluxControlNet(base_cfg, sd, "cpu")
    ref = ref_branch.forward(img, cond, img_ids, txt, txt_ids, t, y, gd)
    dev_branch = C.FluxControlNet(base_cfg, sd, "cuda")
    cu = lambda x: x.cuda().bfloat16() if x.is_floating_point() else x.cuda()                 # noqa: E731
    got = dev_branch.forward(cu(img), cu(cond), img_ids.cuda(), cu(txt), txt_ids.cuda(), t.cuda(), cu(y), gd.cuda())
    assert len(got) == 2
    for a, b in zip(got, ref):
        assert (a.float().cpu() - b).abs().max().item() < 0.06 * max(1.0, b.abs().max().item())
    bw = random_flux_weights(base_cfg, 2, std=0.05)
    want = C.ControlledDit(OracleFluxDiT(base_cfg, bw), ref_branch, cond, 0.7).forward(img, img_ids, txt, txt_ids, t, y, gd)
    base = FluxDiTGpu(base_cfg).load_state_dict(bw)
    out = C.ControlledDit(base, dev_branch, cu(cond), 0.7).forward_graphed(cu(img), img_ids.cuda(), cu(txt), txt_ids.cuda(), t.cuda(),
                                                                         cu(y), gd.cuda())
    assert base.injector is None
    assert (out.float().cpu() - want).abs().max().item() < 0.06 * max(1.0, want.abs().max().item())


def test_flux_ip_adapter_seam_on_device_tracks_the_oracle():
    """The IP-Adapter on the sm_100a model: the image query handed to the seam is the normalised, un-rotated query (its
    own norm launch next to the fused norm + rotation), and the adapted forward tracks the fp32 twin; scale 0 leaves
    the device forward unchanged."""
    from inference_b200.media import flux_ip as P
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT, make_ids, random_flux_weights

    cfg = FluxConfig.tiny()
    bw = random_flux_weights(cfg, 2, std=0.05)
    g = torch.Generator().manual_seed(0)
    ht, wt, St = 8, 8, 16
    img, txt = torch.randn(1, ht * wt, cfg.in_channels, generator=g), torch.randn(1, St, cfg.context_in_dim, generator=g)
    y = torch.randn(1, cfg.vec_in_dim, generator=g)
    txt_ids, img_ids = make_ids(ht, wt, St)
    t, gd = torch.tensor([0.6]), torch.tensor([3.5])
    aw = P.random_ip_adapter_weights(cfg.depth, cfg.hidden_size, 24, seed=4)
    emb = torch.randn(1, 24, generator=g)
    ref_ad = P.FluxIpAdapter(aw, "cpu")
    oracle = OracleFluxDiT(cfg, bw)
    oracle.injector = P.FluxIpInjector(ref_ad, ref_ad.tokens(emb), 0.7)
    want = oracle.forward(img, img_ids, txt, txt_ids, t, y, gd)
    oracle.injector = None
    plain = oracle.forward(img, img_ids, txt, txt_ids, t, y, gd)
    assert (want - plain).abs().max().item() > 1e-3
    dev_ad = P.FluxIpAdapter(aw, "cuda")
    model = FluxDiTGpu(cfg).load_state_dict(bw)
    cu = lambda x: x.cuda().bfloat16() if x.is_floating_point() else x.cuda()                 # noqa: E731
    args = (cu(img), img_ids.cuda(), cu(txt), txt_ids.cuda(), t.cuda(), cu(y), gd.cuda())
    base_out = model.forward(*args).float().cpu()
    model.injector = P.FluxIpInjector(dev_ad, dev_ad.tokens(emb), 0.7)
    got = model.forward(*args).float().cpu()
    model.injector = P.FluxIpInjector(dev_ad, dev_ad.tokens(emb), 0.0)
    off = model.forward(*args).float().cpu()
    model.injector = None
    tol = 0.06 * max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() < tol and (base_out - plain).abs().max().item() < tol
    assert torch.equal(off, base_out)
    assert ((got - base_out) - (want - plain)).abs().max().item() < tol           # the adapter's effect itself agrees


def test_pid_network_on_device_tracks_the_oracle():
    """The PiD network on the sm_100a backend (bf16 projections on the tcgen05 GEMM, 64-wide-head attention on the 64-wide
    attention kernel, fp32 adapter trunk) against the fp32 backend carrying the same weights, v1.5 adapter."""
    from inference_b200.media import pid as P

    cfg = P.PidConfig(num_groups=2, hidden_size=128, pixel_hidden_size=8, pixel_attn_hidden_size=128, pixel_num_groups=2, patch_depth=3,
                      pixel_depth=1, patch_size=4, txt_embed_dim=32, txt_max_length=12, rope_ref_h=32, rope_ref_w=32,
                      lq_latent_channels=4, lq_hidden_dim=16, lq_num_res_blocks=1, lq_interval=2, sr_scale=2,
                      latent_spatial_down_factor=8, lq_replicate_padding=True, pit_lq_inject=True)
    w = P.random_pid_weights(cfg, seed=1)
    g = torch.Generator().manual_seed(0)
    x, y = torch.randn(1, 3, 64, 64, generator=g), torch.randn(1, 12, 32, generator=g)
    lq, t, sig = torch.randn(1, 4, 4, 4, generator=g), torch.tensor([634.0]), torch.tensor([0.3])
    want = P.PidNet(w, cfg, "cpu").forward(x, t, y, lq, sig)
    got = P.PidNet(w, cfg, "cuda").forward(x, t, y, lq, sig).float().cpu()
    assert got.shape == want.shape == (1, 3, 64, 64)
    assert (got - want).abs().max().item() < 0.08 * max(1.0, want.abs().max().item())
    assert float((got - want).abs().mean()) / (float(want.abs().mean()) + 1e-6) < 0.05
