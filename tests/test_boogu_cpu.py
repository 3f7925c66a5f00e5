"""Boogu-Image: schedules, chat rendering, rotary position layout, the hybrid DiT against an independent restatement of
one block of each kind, and the three providers on a synthetic snapshot (text -> image, image -> image, the turbo
re-noising loop, multi-reference edit)."""
import math

import pytest
import torch
import torch.nn.functional as F

from inference_b200.media import boogu as B
from inference_b200.models import dit_boogu as D


def test_schedules_and_chat():
    assert B.lin_mu() == pytest.approx(1.15) and B.lin_mu(256.0) == pytest.approx(0.5)
    s = B.base_sigmas(4)
    assert len(s) == 5 and s[0] == pytest.approx(1.0, abs=1e-6) and s[-1] == 0.0 and all(a > b for a, b in zip(s, s[1:]))
    # t = 0.5 under mu: 1 - e^mu / (e^mu + 1)
    assert 1.0 - s[2] == pytest.approx(1.0 - math.exp(1.15) / (math.exp(1.15) + 1.0))
    assert B.dmd_levels(4) == pytest.approx([0.001, 0.25075, 0.5005, 0.75025])
    assert B.turbo_sigmas(4) == pytest.approx([0.999, 0.74925, 0.4995, 0.24975, 0.0])
    assert B.render_chat("S", "U") == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n"
    assert B.render_chat("S", "U", [2, 1]) == ("<|im_start|>system\nS<|im_end|>\n<|im_start|>user\n<|vision_start|><|image_pad|>"
                                               "<|image_pad|><|vision_end|><|vision_start|><|image_pad|><|vision_end|>U<|im_end|>\n")


def test_rope_positions_layout():
    pos = D.rope_positions(3, [(2, 2), (3, 1)], 4, 4)
    assert pos.shape == (3 + 4 + 3 + 16, 3)
    assert pos[2].tolist() == [2.0, 2.0, 2.0]
    assert pos[3].tolist() == [3.0, 0.0, 0.0] and pos[6].tolist() == [3.0, 1.0, 1.0]           # first reference at t = cap
    assert pos[7].tolist() == [5.0, 0.0, 0.0] and pos[9].tolist() == [5.0, 2.0, 0.0]           # second at cap + max(2, 2)
    assert pos[10].tolist() == [8.0, 0.0, 0.0] and pos[-1].tolist() == [8.0, 3.0, 3.0]         # image at cap + 2 + max(3, 1)
    t2i = D.rope_positions(5, [], 2, 3)
    assert t2i[5].tolist() == [5.0, 0.0, 0.0] and t2i[-1].tolist() == [5.0, 1.0, 2.0]


def _cfg():
    return D.BooguConfig.from_json(dict(hidden_size=48, num_layers=2, num_double_stream_layers=1, num_refiner_layers=1,
                                        num_attention_heads=4, num_kv_heads=2, axes_dim_rope=[4, 4, 4], text_dim=20, multiple_of=16))


def test_config_rules():
    assert D.BooguConfig().head_dim == 120 and D.BooguConfig().num_single_stream_layers == 32 and D.ffn_dim(D.BooguConfig()) == 8960
    with pytest.raises(ValueError, match="head_dim"):
        D.BooguConfig.from_json(dict(hidden_size=48, num_attention_heads=4, num_kv_heads=2, axes_dim_rope=[4, 4, 2]))
    with pytest.raises(ValueError, match="num_kv_heads"):
        D.BooguConfig.from_json(dict(hidden_size=48, num_attention_heads=4, num_kv_heads=3, axes_dim_rope=[4, 4, 4]))
    with pytest.raises(ValueError, match="reduce_type"):
        D.BooguConfig.from_json(dict(instruction_feature_configs={"reduce_type": "max"}))


def test_blocks_match_a_restatement():
    cfg = _cfg()
    w = D.random_boogu_weights(cfg, 2)
    dit = D.BooguDiT(cfg, w)
    H, K, hd = 4, 2, 12
    torch.manual_seed(0)
    lin = lambda x, p: F.linear(x, w[p + ".weight"], w.get(p + ".bias"))                        # noqa: E731
    rms = lambda x, g, eps=cfg.norm_eps: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g   # noqa: E731
    S = 7
    ang = torch.rand(S, hd // 2) * 3
    cos, sin = ang.cos(), ang.sin()

    def rope(x):                                   # [1, S, h, hd]
        a, b = x[..., 0::2], x[..., 1::2]
        c, s = cos[None, :, None], sin[None, :, None]
        return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)

    def attn(x, p):
        q = rope(rms(lin(x, p + ".to_q").view(1, S, H, hd), w[p + ".norm_q.weight"], 1e-5)).transpose(1, 2)
        k = rope(rms(lin(x, p + ".to_k").view(1, S, K, hd), w[p + ".norm_k.weight"], 1e-5)).transpose(1, 2)
        v = lin(x, p + ".to_v").view(1, S, K, hd).transpose(1, 2)
        k, v = k.repeat_interleave(H // K, 1), v.repeat_interleave(H // K, 1)
        o = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(hd), -1) @ v
        return lin(o.transpose(1, 2).reshape(1, S, H * hd), p + ".to_out.0")

    def swiglu(x, p):
        return lin(F.silu(lin(x, p + ".linear_1")) * lin(x, p + ".linear_3"), p + ".linear_2")

    x, temb = torch.randn(1, S, 48), torch.randn(1, 1, 48)
    p = "context_refiner.0"
    y = x + rms(attn(rms(x, w[p + ".norm1.weight"]), p + ".attn"), w[p + ".norm2.weight"])
    want = y + rms(swiglu(rms(y, w[p + ".ffn_norm1.weight"]), p + ".feed_forward"), w[p + ".ffn_norm2.weight"])
    assert torch.allclose(dit._plain_block(x, p, (cos, sin)), want, atol=1e-5)
    p = "noise_refiner.0"
    a, b, c, d = lin(F.silu(temb), p + ".norm1.linear").chunk(4, -1)
    y = x + torch.tanh(b) * rms(attn(rms(x, w[p + ".norm1.norm.weight"]) * (1 + a), p + ".attn"), w[p + ".norm2.weight"])
    want = y + torch.tanh(d) * rms(swiglu(rms(y, w[p + ".ffn_norm1.weight"]) * (1 + c), p + ".feed_forward"), w[p + ".ffn_norm2.weight"])
    assert torch.allclose(dit._mod_block(x, p, (cos, sin), F.silu(temb)), want, atol=1e-5)


def test_forward_shapes_and_reference_sensitivity():
    cfg = _cfg()
    dit = D.BooguDiT(cfg, D.random_boogu_weights(cfg, 3))
    torch.manual_seed(1)
    z, ins = torch.randn(1, 16, 8, 12), torch.randn(1, 5, 20)
    t = torch.tensor([0.3])
    v = dit.forward(z, t, ins)
    assert v.shape == z.shape and torch.isfinite(v).all()
    assert torch.equal(dit.forward(z, t, ins), v)
    r = torch.randn(1, 16, 4, 6)
    ve = dit.forward(z, t, ins, (r,))
    assert ve.shape == z.shape and not torch.allclose(ve, v, atol=1e-4)
    assert not torch.allclose(dit.forward(z, t, ins, (r, r)), ve, atol=1e-5)           # the index embedding and position move
    assert not torch.allclose(dit.forward(z, torch.tensor([0.8]), ins), v, atol=1e-4)
    # patchify / unpatchify are inverse and ordered (row, column, channel) inside a patch
    assert torch.equal(dit.unpatchify(dit.patchify(z), 4, 6), z)
    assert dit.patchify(z)[0, 0, :16].tolist() == z[0, :, 0, 0].tolist()


def test_providers(tmp_path):
    from inference_b200.contracts.errors import InferenceError
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec
    from inference_b200.contracts.gen_core.generator import Conditioning, ConditioningKind
    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.contracts.gen_core.runtime import ProgressStep
    from inference_b200.media.catalog import provider_registry
    from inference_b200.testkit.generator import Profile, conformance

    snap = B.write_synthetic_snapshot(tmp_path / "boogu")
    reg = provider_registry("cpu")
    for mid in ("cpu_boogu_image", "cpu_boogu_image_turbo", "cpu_boogu_image_edit"):
        assert mid in reg.ids()
    base = reg.load("cpu_boogu_image", LoadSpec.from_dir(snap))
    d = base.descriptor()
    assert d.capabilities.supports_guidance and not d.capabilities.supports_negative_prompt
    assert ConditioningKind.REFERENCE in d.capabilities.conditioning
    conformance(base, Profile(width=256, height=256, steps=2))
    turbo = reg.load("cpu_boogu_image_turbo", LoadSpec.from_dir(snap))
    td = turbo.descriptor()
    assert not td.capabilities.supports_guidance and td.capabilities.samplers == B.TURBO_SAMPLERS
    req = GenerationRequest(prompt="a red fox", width=256, height=256, seed=5)
    ev = []
    out = turbo.generate(req, ev.append)
    assert [(e.current, e.total) for e in ev if isinstance(e, ProgressStep)] == [(i, 4) for i in range(1, 5)]
    assert turbo.generate(req).images[0].pixels == out.images[0].pixels
    sampled = turbo.generate(GenerationRequest(**{**req.__dict__, "sampler": "lcm"}))
    assert sampled.images[0].pixels != out.images[0].pixels
    img = Image(width=64, height=64, pixels=bytes((i * 5) % 256 for i in range(64 * 64 * 3)))
    i2i = base.generate(GenerationRequest(**{**req.__dict__, "steps": 4, "guidance": 1.0,
                                             "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=img, strength=0.5)]}), ev.append)
    t2i = base.generate(GenerationRequest(**{**req.__dict__, "steps": 4, "guidance": 1.0}))
    assert i2i.images[0].pixels != t2i.images[0].pixels
    with pytest.raises(InferenceError):
        base.validate(GenerationRequest(**{**req.__dict__, "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=img)] * 2}))
    with pytest.raises(InferenceError):
        base.validate(GenerationRequest(**{**req.__dict__, "prompt": "   "}))
    with pytest.raises(InferenceError):
        base.validate(GenerationRequest(**{**req.__dict__, "width": 264}))
    edit = reg.load("cpu_boogu_image_edit", LoadSpec.from_dir(snap))
    with pytest.raises(InferenceError, match="at least one"):
        edit.validate(req)
    six = [Conditioning(ConditioningKind.MULTI_REFERENCE, images=[img] * 6)]
    with pytest.raises(InferenceError, match="at most 5"):
        edit.validate(GenerationRequest(**{**req.__dict__, "conditioning": six}))
    odd = Image(width=40, height=64, pixels=bytes(40 * 64 * 3))
    with pytest.raises(InferenceError, match="multiples of 16"):
        edit.validate(GenerationRequest(**{**req.__dict__, "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=odd)]}))
    small = Image(width=32, height=48, pixels=bytes((i * 3) % 256 for i in range(32 * 48 * 3)))
    e1 = edit.generate(GenerationRequest(**{**req.__dict__, "steps": 2, "conditioning": [Conditioning(ConditioningKind.REFERENCE, image=img)]}))
    e2 = edit.generate(GenerationRequest(**{**req.__dict__, "steps": 2,
                                            "conditioning": [Conditioning(ConditioningKind.MULTI_REFERENCE, images=[img, small])]}))
    assert len(e1.images) == 1 and e1.images[0].pixels != e2.images[0].pixels


def test_image_grounded_instruction_matches_hugging_face():
    transformers = pytest.importorskip("transformers")
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.models import qwen3_vl as V
    from inference_b200.models.text_encoders import CausalLmTextEncoder

    cfg = Qwen3VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, vocab_size=200, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True}, tie_word_embeddings=False),
        vision_config=dict(depth=4, hidden_size=48, num_heads=4, intermediate_size=96, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1, 2]),
        image_token_id=150, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153)
    torch.manual_seed(0)
    model = Qwen3VLForConditionalGeneration(cfg).eval()
    sd = dict(model.state_dict())
    lcfg = V.language_model_config(cfg.to_dict())
    lmw = {"model." + k[len("model.language_model."):]: v for k, v in sd.items() if k.startswith("model.language_model.")}
    lm = CausalLmTextEncoder(lcfg, lmw, "cpu", skip_last=0, final_norm=True)
    vc = V.Qwen3VlVisionConfig.from_json(cfg.to_dict())
    imgs = [Image(width=24, height=16, pixels=bytes((i * 7) % 256 for i in range(24 * 16 * 3))),
            Image(width=16, height=16, pixels=bytes((i * 11) % 256 for i in range(16 * 16 * 3)))]
    counts = [(16 // 4) * (24 // 4) // 4, (16 // 4) * (16 // 4) // 4]

    class Tok:
        def encode(self, text, add_special_tokens=False):
            ids = [7, 8, 152] + [150] * counts[0] + [153, 152] + [150] * counts[1] + [153, 9, 10, 11]
            return type("E", (), {"ids": ids})()

    enc = B.BooguInstructionEncoder(lm, Tok(), sd, vc, "cpu", image_token_id=150)
    enc.image_limits = dict(min_pixels=16, max_pixels=10 ** 6)
    got = enc.encode_edit("swap the sky", imgs)
    patches, grids = [], []
    for im in imgs:
        rgb = torch.frombuffer(bytearray(im.pixels), dtype=torch.uint8).view(im.height, im.width, 3)
        p, g = V.image_to_patches(rgb, vc, min_pixels=16, max_pixels=10 ** 6)
        patches.append(p)
        grids.append(g)
    ids = torch.tensor([Tok().encode("").ids])
    with torch.no_grad():
        ref = model.model(input_ids=ids, pixel_values=torch.cat(patches), image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=(ids == 150).int()).last_hidden_state
    assert got.shape == ref.shape
    torch.testing.assert_close(got, ref, atol=3e-4, rtol=1e-3)
    # without a vision tower the edit encoder refuses
    with pytest.raises(B.LoadError):
        B.BooguInstructionEncoder(lm, Tok()).encode_edit("x", imgs)
