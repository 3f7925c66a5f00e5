"""SCAIL-2: colour-class mask compression, windowing, history pinning, the rotary chunks (offsets, lane split, pose
averaging), token packing of the DiT (only the target comes back; every conditioning input matters), the CLIP tower, and the
provider on a synthetic snapshot including a two-window render."""
import pytest
import torch

from inference_b200.media import scail2 as S
from inference_b200.models import dit_scail2 as D


def test_mask_compression():
    m = torch.full((3, 1, 8, 8), -1.0)
    m[0] = 1.0                                                         # red
    out = S.compress_mask_to_latent(m)
    assert out.shape == (28, 1, 1, 1)
    v = out.flatten()
    assert v[1] == 1.0 and v[0] == 0.0 and v[8] == 1.0                 # class 1 (red) in each of the 4 sub-frame groups
    m5 = torch.full((3, 5, 16, 8), -1.0)
    m5[:, 1:] = 1.0                                                    # frames 1.. white, frame 0 black
    m5[1, 3, :8] = -1.0                                                # frame 3: top half magenta (r, b on, g off)
    out = S.compress_mask_to_latent(m5)
    assert out.shape == (28, 2, 2, 1)
    assert out[:, 0].abs().max() == 0.0                                # latent frame 0 = first frame x 4: no class
    assert out[0, 1, 0, 0] == 1.0 and out[2 * 7 + 0, 1, 0, 0] == 0.0 and out[2 * 7 + 5, 1, 0, 0] == 1.0 and out[2 * 7 + 0, 1, 1, 0] == 1.0
    for bad, msg in ((torch.zeros(3, 1, 7, 8), "divisible by 8"), (torch.zeros(3, 3, 8, 8), "divisible by temporal_stride")):
        with pytest.raises(S.InferenceError, match=msg):
            S.compress_mask_to_latent(bad)


def test_windows_and_history():
    assert S.build_segments(81) == [(0, 81)] and S.build_segments(50) == [(0, 49)] and S.build_segments(0) == []
    segs = S.build_segments(200)
    assert segs == [(0, 81), (76, 157), (152, 197)]
    for s, e in segs:
        assert (e - s - 1) % 4 == 0
    assert S.build_segments(160) == [(0, 81), (76, 157)]              # a 8-frame tail aligns to 5 = the overlap: dropped
    assert S.vae_align(6) == 5 and S.align(100) == 96 and S.align(10) == 32
    lat, hist = torch.zeros(2, 4, 1, 1), torch.ones(2, 2, 1, 1)
    assert S.apply_clean_history(lat, hist)[:, :, 0, 0].tolist() == [[1.0, 1.0, 0.0, 0.0]] * 2
    assert S.apply_clean_history(lat, None) is lat
    x = torch.tensor([[[[1.0, 3.0], [5.0, 7.0]]]])
    assert S.downsample_half(x).item() == pytest.approx(4.0)


def test_rotary_chunks():
    r = D.ScailRope(128)
    assert (r.inv_t.numel(), r.inv_a.numel(), r.half_d) == (22, 21, 64)
    cos, sin = r.chunk((2, 3, 4))
    assert cos.shape == (24, 64) and torch.allclose(cos[0], torch.ones(64)) and torch.allclose(sin[0], torch.zeros(64))
    c2, _ = r.chunk((1, 3, 4), (5, 2, 0))
    tok = 1 * 4 + 3                                                    # row 1, column 3
    assert c2[tok, 0] == pytest.approx(torch.cos(torch.tensor(5.0)).item(), abs=1e-6)
    assert c2[tok, 22] == pytest.approx(torch.cos(torch.tensor(3.0)).item(), abs=1e-6)         # row 1 + shift 2
    assert c2[tok, 43] == pytest.approx(torch.cos(torch.tensor(3.0)).item(), abs=1e-6)         # column 3
    cp, sp = r.chunk((1, 4, 4), (0, 0, 120), pose_downsample=True)
    full_c, _ = r.chunk((1, 4, 4), (0, 0, 120))
    assert cp.shape == (4, 64)
    assert torch.allclose(cp[1], full_c.view(4, 4, 64)[0:2, 2:4].mean((0, 1)), atol=1e-6)


def _tiny():
    cfg = D.Scail2Config.from_json(dict(dim=256, ffn_dim=128, num_heads=2, num_layers=2, text_dim=16, text_len=8, clip_dim=32, freq_dim=32))
    return cfg, D.Scail2DiT(cfg, D.random_scail2_weights(cfg, 1))


def test_token_packing_and_sensitivity():
    cfg, dit = _tiny()
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    x, ref, rm, pose, dm = rn(16, 2, 4, 4), rn(16, 1, 4, 4), torch.rand(28, 3, 4, 4, generator=g), rn(16, 2, 2, 2), torch.rand(28, 2, 2, 2, generator=g)
    txt, img = dit.embed_text(rn(5, 16)), dit.embed_img(rn(1, 5, 32))
    assert txt.shape == (1, 8, 256) and img.shape == (1, 5, 256)
    base = dit.forward(x, ref, rm, pose, dm, txt, img, 700.0)
    assert base.shape == (16, 2, 4, 4) and torch.isfinite(base).all()
    differs = lambda o: not torch.allclose(o, base, atol=1e-4)        # noqa: E731
    assert differs(dit.forward(x, ref + 1, rm, pose, dm, txt, img, 700.0))
    assert differs(dit.forward(x, ref, rm, pose + 1, dm, txt, img, 700.0))
    assert differs(dit.forward(x, ref, rm, pose, 1 - dm, txt, img, 700.0))
    assert differs(dit.forward(x, ref, rm, pose, dm, txt, dit.embed_img(rn(1, 5, 32)), 700.0))
    assert differs(dit.forward(x, ref, rm, pose, dm, txt, img, 700.0, replace_flag=True))
    assert differs(dit.forward(x, ref, rm, pose, dm, txt, img, 700.0, history_mask=torch.ones(4, 2, 4, 4)))
    extra = dit.forward(x, ref, rm, pose, dm, txt, img, 700.0, additional_ref_latent=rn(16, 2, 4, 4), additional_ref_masks=torch.rand(28, 2, 4, 4, generator=g))
    assert extra.shape == base.shape and differs(extra)
    with pytest.raises(ValueError):
        dit.forward(x, ref, rm, pose, dm, txt, img, 700.0, additional_ref_latent=rn(16, 1, 4, 4))
    tok, grid = D.patchify(x, (1, 2, 2))
    assert grid == (2, 2, 2) and tok.shape == (8, 64) and tok[0, :4].tolist() == x[0, 0, :2, :2].flatten().tolist()
    back = D.unpatchify(torch.arange(8 * 64.0).view(8, 64), grid, 16, (1, 2, 2))
    assert back.shape == (16, 2, 4, 4) and back[3, 0, 0, 1] == 0 * 64 + 1 * 16 + 3       # token 0, patch offset (0, 1), channel 3


def test_clip_tower():
    cfg = D.ClipVisionConfig(image_size=28, patch_size=14, dim=32, num_heads=2, num_layers=3, mlp_dim=64)
    clip = D.ScailClip(cfg, D.random_clip_weights(cfg, 2))
    out = clip.encode(torch.randn(1, 3, 28, 28))
    assert out.shape == (1, 5, 32) and torch.isfinite(out).all()
    assert len([k for k in clip.w.w if k.startswith("transformer.")]) == 2 * 12            # the last block is not stored / run
    px = S.clip_preprocess(torch.zeros(3, 10, 12), 28)
    assert px.shape == (1, 3, 28, 28) and px[0, 0, 0, 0] == pytest.approx((0.5 - S.CLIP_MEAN[0]) / S.CLIP_STD[0])


def test_provider(tmp_path):
    from inference_b200.contracts.errors import InferenceError, LoadError, Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressDecoding, ProgressStep
    from inference_b200.media.catalog import provider_registry

    snap = S.write_synthetic_snapshot(tmp_path / "scail2")
    reg = provider_registry("cpu")
    assert "cpu_scail2_14b" in reg.ids()
    with pytest.raises(LoadError, match="does not exist"):
        reg.load("cpu_scail2_14b", LoadSpec.from_dir(tmp_path / "nope"))
    gen = reg.load("cpu_scail2_14b", LoadSpec.from_dir(snap))
    d = gen.descriptor()
    assert d.family == "scail2" and d.capabilities.supports_lora and d.capabilities.supports_lokr and "unipc" in d.capabilities.samplers
    assert ConditioningKind.MULTI_REFERENCE not in d.capabilities.conditioning
    img = lambda k, w=64, h=64: Image(w, h, bytes((i * k) % 256 for i in range(w * h * 3)))          # noqa: E731
    clip = Conditioning(ConditioningKind.CONTROL_CLIP, frames=[img(k) for k in (3, 5, 7, 11, 13)], mask_frames=[img(k + 1) for k in (3, 5, 7, 11, 13)])
    cond = [Conditioning(ConditioningKind.REFERENCE, image=img(17)), Conditioning(ConditioningKind.MASK, image=img(19)), clip]
    req = GenerationRequest(prompt="a dancer", width=64, height=64, steps=2, seed=3, guidance=2.0, conditioning=cond, sampler="euler")
    ev = []
    out = gen.generate(req, ev.append)
    assert len(out.video_frames) == 5 and out.fps == 16 and (out.video_frames[0].width, out.video_frames[0].height) == (64, 64)
    assert [(e.current, e.total) for e in ev if isinstance(e, ProgressStep)] == [(1, 2), (2, 2)] and any(isinstance(e, ProgressDecoding) for e in ev)
    rep = gen.generate(GenerationRequest(**{**req.__dict__, "video_mode": "replacement"}))
    assert rep.video_frames[2].pixels != out.video_frames[2].pixels
    for drop in (0, 1, 2):
        with pytest.raises(InferenceError):
            gen.generate(GenerationRequest(**{**req.__dict__, "conditioning": [c for j, c in enumerate(cond) if j != drop]}))
    with pytest.raises(Unsupported):
        gen.validate(GenerationRequest(**{**req.__dict__, "conditioning": cond + [Conditioning(ConditioningKind.MULTI_REFERENCE, images=[img(2)])]}))
    with pytest.raises(InferenceError):
        gen.validate(GenerationRequest(**{**req.__dict__, "steps": 0}))
    # two windows: 9 frames in windows of 5 overlapping by 1 -> frames 0-4, then 4-8 with frame 4 pinned as history
    pipe = gen.pipe
    heavy, text = pipe.load_heavy(), pipe.load_text()
    long_clip = Conditioning(ConditioningKind.CONTROL_CLIP, frames=[img(k) for k in range(3, 12)], mask_frames=[img(k + 1) for k in range(3, 12)])
    lreq = GenerationRequest(**{**req.__dict__, "conditioning": cond[:2] + [long_clip], "steps": 1, "guidance": 1.0})
    ev2 = []
    frames = pipe.render(heavy, pipe.encode(text, lreq), lreq, ev2.append, segment_len=5, overlap=1)
    assert len(frames) == 9 and [(e.current, e.total) for e in ev2 if isinstance(e, ProgressStep)] == [(1, 2), (2, 2)]
