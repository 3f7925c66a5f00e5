"""Bernini renderer: mode resolution, knobs, source-id rotary phase, packed-token velocity, the guidance algebra
(chains and adaptive projected guidance) and the generator surface on a synthetic two-expert snapshot."""
import math

import pytest
import torch

from inference_b200.media import bernini as B
from inference_b200.models.dit_wan import WanConfig, WanDiT, random_wan_weights


def test_mode_resolution_and_conditioning_rules():
    assert B.resolve_mode("rv2v", False, False) is B.Mode.RV2V
    assert B.resolve_mode("t2v_apg", False, False) is B.Mode.T2V_APG
    assert B.resolve_mode("t2i", False, False) is B.Mode.T2V_APG
    assert B.resolve_mode("r2v", False, True) is B.Mode.R2V_APG
    assert B.resolve_mode(None, False, False) is B.Mode.T2V_APG
    assert B.resolve_mode(None, True, False) is B.Mode.V2V_APG
    assert B.resolve_mode(None, False, True) is B.Mode.V2V
    assert B.resolve_mode(None, True, True) is B.Mode.RV2V
    assert B.resolve_mode("t2v", False, False) is B.Mode.T2V
    assert not B.Mode.T2V.needs_conditioning and not B.Mode.T2V_APG.needs_conditioning
    assert all(m.needs_conditioning for m in (B.Mode.V2V, B.Mode.V2V_CHAIN, B.Mode.V2V_APG, B.Mode.R2V_APG, B.Mode.RV2V))
    assert B.Mode.T2V_APG.is_apg and not B.Mode.T2V.is_apg
    for mode, src, ok in ((B.Mode.V2V_APG, False, False), (B.Mode.RV2V, False, False), (B.Mode.V2V_APG, True, True),
                          (B.Mode.T2V_APG, False, True), (B.Mode.T2V, False, True), (B.Mode.T2V_APG, True, False)):
        if ok:
            B.check_mode_conditioning("id", mode, src)
        else:
            with pytest.raises(B.InferenceError):
                B.check_mode_conditioning("id", mode, src)


def test_knobs(tmp_path):
    k = B.BerniniKnobs.from_dir(tmp_path)
    assert (k.switch_dit_boundary, k.shift, k.max_trained_src_id, k.max_sequence_length) == (0.875, 3.0, 5.0, 512)
    (tmp_path / "bernini_renderer.json").write_text('{"shift": 4.5, "interpolate_src_id": false}')
    k = B.BerniniKnobs.from_dir(tmp_path)
    assert k.shift == 4.5 and k.interpolate_src_id is False and k.switch_dit_boundary == 0.875
    (tmp_path / "bernini_renderer.json").write_text("{ this is not json ]")
    with pytest.raises(B.LoadError, match="bernini_renderer.json"):
        B.BerniniKnobs.from_dir(tmp_path)


def test_source_ids_and_rotary_phase():
    assert B.assign_source_ids(0, 5.0, True) == []
    assert B.assign_source_ids(3, 5.0, True) == [1.0, 2.0, 3.0]
    assert B.assign_source_ids(9, 5.0, True) == pytest.approx([1.0 + 0.5 * i for i in range(9)])
    assert B.assign_source_ids(7, 5.0, False) == [float(i) for i in range(1, 8)]
    ang = torch.rand(6, 4, dtype=torch.float64) * 3
    cos, sin = ang.cos().float(), ang.sin().float()
    c0, s0 = B.apply_source_id(cos, sin, 0.0, 8)
    assert c0 is cos and s0 is sin
    c2, s2 = B.apply_source_id(cos, sin, 2.0, 8)
    want = ang + 2.0 * torch.tensor([10000.0 ** (-2 * k / 8) for k in range(4)], dtype=torch.float64)
    assert torch.allclose(c2, want.cos().float(), atol=1e-6) and torch.allclose(s2, want.sin().float(), atol=1e-6)


def _tiny():
    cfg = WanConfig(num_attention_heads=2, attention_head_dim=128, num_layers=2, ffn_dim=64, text_dim=16, freq_dim=32)
    return cfg, WanDiT(cfg, random_wan_weights(cfg, 1, 0.05))


def test_packed_velocity_and_guidance_modes():
    cfg, dit = _tiny()
    torch.manual_seed(0)
    noisy = torch.randn(1, 16, 2, 4, 4)
    cc, cu = dit.embed_text(torch.randn(1, 3, 16)), dit.embed_text(torch.randn(1, 3, 16))
    pf = B.PackedForward(B.BerniniKnobs())
    # without sources the packed path is the plain forward
    plain = dit.forward(noisy, torch.full((1,), 833.0), cc, embedded=True).float()
    assert torch.allclose(pf.velocity(dit, noisy, [], 833.0, cc), plain, atol=1e-5)
    img = torch.randn(1, 16, 1, 4, 4)
    v1 = pf.velocity(dit, noisy, [(img, 1.0)], 833.0, cc)
    assert v1.shape == noisy.shape and not torch.allclose(v1, plain, atol=1e-4)
    assert torch.equal(pf.velocity(dit, noisy, [(img, 1.0)], 833.0, cc), v1)                       # warm token cache
    assert torch.equal(B.PackedForward(B.BerniniKnobs()).velocity(dit, noisy, [(img, 1.0)], 833.0, cc), v1)
    assert not torch.allclose(pf.velocity(dit, noisy, [(img, 2.0)], 833.0, cc), v1, atol=1e-5)    # the source id matters
    g = B.GuidanceParams(omega_vid=1.0, omega_img=1.0, omega_txt=4.0)
    eu, ec = pf.velocity(dit, noisy, [], 833.0, cu), pf.velocity(dit, noisy, [], 833.0, cc)
    got = B.guided_velocity(pf, B.Mode.T2V, dit, noisy, [], [], 833.0, 1.0, cc, cu, g, [])
    assert torch.allclose(got, eu + (ec - eu) * 4.0, atol=1e-6)
    # APG with eta = 1 and no clipping is plain CFG in sample space, hence in velocity space
    g1 = B.GuidanceParams(omega_txt=4.0, eta=1.0, norm_threshold=(0.0, 0.0))
    apg = B.guided_velocity(pf, B.Mode.T2V_APG, dit, noisy, [], [], 833.0, 0.7, cc, cu, g1, [B.MomentumBuffer(0.0)])
    assert torch.allclose(apg, eu + (ec - eu) * 4.0, atol=1e-4)
    vid = torch.randn(1, 16, 2, 4, 4)
    for mode, nb in ((B.Mode.V2V, 0), (B.Mode.V2V_CHAIN, 0), (B.Mode.RV2V, 0), (B.Mode.V2V_APG, 1), (B.Mode.R2V_APG, 2)):
        assert B.num_momentum_buffers(mode) == nb
        out = B.guided_velocity(pf, mode, dit, noisy, [vid], [img], 500.0, 0.5, cc, cu, g, [B.MomentumBuffer(0.0) for _ in range(nb)])
        assert out.shape == noisy.shape and torch.isfinite(out).all()
    combos = pf.combos([vid, vid * 2], [])
    assert len(combos["v"]) == 2 and combos["v"][1][1] == combos["vi"][1][1] == 2.0 and pf.combos([], [])["v"] == []


def test_normalized_guidance_properties():
    det = lambda s: (((torch.arange(32, dtype=torch.float32) * 7.0 + s * 13.0) % 11.0) - 5.0).view(1, 4, 2, 2, 2)   # noqa: E731
    cond, uncond = det(1.0), det(2.0)
    got = B.normalized_guidance(cond, uncond, 4.0, None, 1.0, 0.0)
    assert torch.allclose(got, uncond + (cond - uncond) * 4.0, atol=1e-4)
    buf = B.MomentumBuffer(0.5)
    B.normalized_guidance(det(3.0), uncond, 3.0, buf, 0.8, 0.0)
    hist = B.normalized_guidance(det(4.0), uncond, 3.0, buf, 0.8, 0.0)
    fresh = B.normalized_guidance(det(4.0), uncond, 3.0, None, 0.8, 0.0)
    assert (hist - fresh).abs().max() > 1e-4
    # clipping: the per-frame norm of the applied difference never exceeds the threshold (eta = 1 keeps it whole)
    d = B._normalize_diff(cond - uncond, cond, None, 1.0, 1.5)
    assert (d.pow(2).sum((1, 3, 4)).sqrt() <= 1.5 + 1e-5).all()
    # eta = 0 leaves nothing along the conditional direction
    d0 = B._normalize_diff(cond - uncond, cond, None, 0.0, 0.0)
    assert (d0 * cond).sum((1, 3, 4)).abs().max() < 1e-3
    out = B.normalized_guidance_chain(uncond, [det(3.0), det(4.0)], [2.0, 5.0], [B.MomentumBuffer(0.3), B.MomentumBuffer(0.3)], 0.6, [1.0, 0.0])
    assert out.shape == cond.shape
    with pytest.raises(B.InferenceError):
        B.normalized_guidance_chain(uncond, [det(3.0)], [2.0, 5.0], [B.MomentumBuffer(0.3)], 0.6, [1.0])


def test_generator_surface(tmp_path):
    from inference_b200.contracts.errors import InferenceError, LoadError, Unsupported
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind, Modality
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressStep, WeightsSource
    from inference_b200.media.catalog import provider_registry

    snap = B.write_synthetic_snapshot(tmp_path / "b")
    reg = provider_registry("cpu")
    assert "cpu_bernini_renderer" in reg.ids()
    gen = reg.load("cpu_bernini_renderer", LoadSpec.from_dir(snap))
    d = gen.descriptor()
    assert d.family == "bernini" and d.modality is Modality.VIDEO and d.capabilities.supports_guidance
    assert "uni_pc" in d.capabilities.samplers and "unipc" in d.capabilities.samplers
    assert {ConditioningKind.REFERENCE, ConditioningKind.MULTI_REFERENCE, ConditioningKind.VIDEO_CLIP} <= set(d.capabilities.conditioning)
    ok = GenerationRequest(prompt="a cat walking across a sunny garden", width=64, height=64, guidance=4.0, frames=5, steps=3, seed=3,
                           sampler="uni_pc")
    gen.validate(ok)
    for bad in (dict(prompt=""), dict(frames=16), dict(width=60), dict(steps=0), dict(video_mode="v2v_apg")):
        with pytest.raises(InferenceError):
            gen.validate(GenerationRequest(**{**ok.__dict__, **bad}))
    events = []
    out = gen.generate(ok, events.append)
    assert len(out.video_frames) == 5 and out.fps == 16 and len(out.video_frames[0].pixels) == 64 * 64 * 3
    assert [(e.current, e.total) for e in events if isinstance(e, ProgressStep)] == [(1, 3), (2, 3), (3, 3)]
    again = gen.generate(ok)
    assert again.video_frames[2].pixels == out.video_frames[2].pixels
    img = Image(width=40, height=32, pixels=bytes((i * 7) % 256 for i in range(40 * 32 * 3)))
    ref = GenerationRequest(**{**ok.__dict__, "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=img)], "sampler": "euler"})
    assert B.resolve_mode(None, False, True) is B.Mode.V2V
    with_ref = gen.generate(ref)
    assert with_ref.video_frames[2].pixels != out.video_frames[2].pixels
    clip = GenerationRequest(**{**ok.__dict__, "frames": 1, "conditioning": [Conditioning(ConditioningKind.VIDEO_CLIP, frames=[img] * 5),
                                                                              Conditioning(ConditioningKind.MULTI_REFERENCE, images=[img, img])]})
    still = gen.generate(clip)
    assert len(still.images) == 1 and not still.video_frames
    with pytest.raises(InferenceError, match="1 \\+ 4k"):
        gen.generate(GenerationRequest(**{**ok.__dict__, "conditioning": [Conditioning(ConditioningKind.VIDEO_CLIP, frames=[img] * 4)]}))
    with pytest.raises(LoadError):
        reg.load("cpu_bernini_renderer", LoadSpec(weights=WeightsSource.file(snap / "swb_config.json")))
