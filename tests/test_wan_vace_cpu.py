"""Wan-VACE: mask unfolding / temporal resampling, the inactive / reactive latent split with reference frames, the control
branch of the DiT (a zero control scale is the plain network; hints land after the configured blocks), and the provider
on a synthetic snapshot."""
import pytest
import torch

from inference_b200.media import wan_vace as V
from inference_b200.models.dit_wan import WanConfig


def test_mask_and_latent_preparation():
    m = torch.tensor([0.0, 0.4, 0.6, 1.0]).view(1, 1, 1, 2, 2)
    assert V.binarize_mask(m).flatten().tolist() == [0.0, 0.0, 1.0, 1.0]
    x = torch.arange(5.0).view(1, 5, 1, 1)
    assert V.nearest_exact_temporal(x, 1, 2).flatten().tolist() == [1.0, 3.0]
    out = V.prepare_masks(torch.ones(1, 3, 5, 32, 32), 2, 1)
    assert out.shape == (1, 64, 3, 4, 4) and float(out[:, :, 0].abs().max()) == 0.0 and float(out[:, :, 1:].min()) == 1.0
    # the unfold puts pixel (dy, dx) of every 8 x 8 cell into channel dy * 8 + dx
    mk = torch.zeros(1, 1, 1, 16, 16)
    mk[0, 0, 0, 9, 3] = 1.0                                  # cell (1, 0), offset (1, 3)
    un = V.prepare_masks(mk, 2, 0)
    assert un.shape == (1, 64, 1, 2, 2) and un[0, 1 * 8 + 3, 0, 1, 0] == 1.0 and un.sum() == 1.0
    enc = lambda v: v[:, :1, ::4, ::8, ::8].repeat(1, 16, 1, 1, 1)              # noqa: E731  a stand-in encoder
    video, mask = torch.rand(1, 3, 5, 16, 16), torch.zeros(1, 3, 5, 16, 16)
    mask[:, :, :, :8] = 1.0
    lat = V.prepare_video_latents(enc, video, mask, [torch.rand(1, 3, 1, 16, 16)])
    assert lat.shape == (1, 32, 3, 2, 2)
    assert float(lat[:, 16:, 0].abs().max()) == 0.0                              # the reference frame has no reactive half
    assert float(lat[:, :16, 1:, 0].abs().max()) == 0.0 and float(lat[:, 16:, 1:, 1].abs().max()) == 0.0   # split by the mask


def test_control_branch():
    cfg = WanConfig(num_attention_heads=2, attention_head_dim=128, num_layers=3, ffn_dim=64, text_dim=16, freq_dim=32)
    w = V.random_vace_weights(cfg, (0, 2), 1)
    dit = V.WanVaceDiT(cfg, w, (0, 2))
    torch.manual_seed(0)
    z, ctx = torch.randn(1, 16, 2, 4, 4), dit.embed_text(torch.randn(1, 3, 16))
    t = torch.full((1,), 700.0)
    ce = dit.embed_control(torch.randn(1, 96, 2, 4, 4), 8)
    assert ce.shape == (1, 8, 256)
    plain = dit.forward(z, t, ctx, embedded=True)
    assert torch.allclose(dit.forward_vace(z, t, ce, ctx, [0.0, 0.0]), plain, atol=1e-6)
    on = dit.forward_vace(z, t, ce, ctx, [1.0, 1.0])
    assert on.shape == z.shape and not torch.allclose(on, plain, atol=1e-4)
    assert not torch.allclose(dit.forward_vace(z, t, ce, ctx, [1.0, 0.0]), on, atol=1e-5)
    with pytest.raises(V.InferenceError, match="scales len"):
        dit.forward_vace(z, t, ce, ctx, [1.0])
    with pytest.raises(V.InferenceError, match="exceeds"):
        dit.embed_control(torch.randn(1, 96, 2, 4, 4), 4)
    assert dit.embed_control(torch.randn(1, 96, 1, 4, 4), 8)[:, 4:].abs().max() == 0.0


def test_provider(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressStep
    from inference_b200.media.catalog import provider_registry

    snap = V.write_synthetic_snapshot(tmp_path / "vace")
    reg = provider_registry("cpu")
    assert "cpu_wan_vace" in reg.ids()
    gen = reg.load("cpu_wan_vace", LoadSpec.from_dir(snap))
    d = gen.descriptor()
    assert d.family == "wan" and ConditioningKind.CONTROL_CLIP in d.capabilities.conditioning
    frame = lambda k: Image(width=64, height=64, pixels=bytes((i * k) % 256 for i in range(64 * 64 * 3)))         # noqa: E731
    white, black = Image(64, 64, bytes([255]) * (64 * 64 * 3)), Image(64, 64, bytes(64 * 64 * 3))
    clip = Conditioning(ConditioningKind.CONTROL_CLIP, frames=[frame(k) for k in (3, 5, 7, 11, 13)], mask_frames=[black, black, white, white, white])
    req = GenerationRequest(prompt="a dancer", width=256, height=256, steps=2, seed=2, guidance=2.0, conditioning=[clip], sampler="euler")
    with pytest.raises(InferenceError, match="ControlClip"):
        gen.validate(GenerationRequest(**{**req.__dict__, "conditioning": []}))
    with pytest.raises(InferenceError, match="4k \\+ 1"):
        gen.validate(GenerationRequest(**{**req.__dict__, "conditioning": [Conditioning(ConditioningKind.CONTROL_CLIP, frames=[white] * 4, mask_frames=[white] * 4)]}))
    with pytest.raises(InferenceError, match="mask frames"):
        gen.validate(GenerationRequest(**{**req.__dict__, "conditioning": [Conditioning(ConditioningKind.CONTROL_CLIP, frames=[white] * 5, mask_frames=[white] * 4)]}))
    small = GenerationRequest(**{**req.__dict__, "width": 256, "height": 256})
    ev = []
    out = gen.generate(small, ev.append)
    assert len(out.video_frames) == 5 and out.fps == 16 and (out.video_frames[0].width, out.video_frames[0].height) == (256, 256)
    assert [(e.current, e.total) for e in ev if isinstance(e, ProgressStep)] == [(1, 2), (2, 2)]
    with_ref = gen.generate(GenerationRequest(**{**small.__dict__, "conditioning": [clip, Conditioning(ConditioningKind.REFERENCE, image=frame(17))]}))
    assert len(with_ref.video_frames) == 5 and with_ref.video_frames[2].pixels != out.video_frames[2].pixels
    weak = gen.generate(GenerationRequest(**{**small.__dict__, "control_scale": 0.0}))
    assert weak.video_frames[2].pixels != out.video_frames[2].pixels
