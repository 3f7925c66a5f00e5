"""gen_core host utilities: checkpoint metadata and adapter key conventions, weight licenses, PIL-exact resampling,
BS.1770 loudness."""
import json
import math

import numpy as np
import pytest
import torch

from inference_b200.contracts.gen_core import audio_dsp, imageops, license as lic, weightsmeta as wm
from inference_b200.contracts.gen_core.media import AudioTrack, Image
from inference_b200.io.safetensors_io import save_file


def test_checkpoint_meta_and_adapter_keys(tmp_path):
    save_file({"a.weight": torch.zeros(4, 8), "b.bias": torch.zeros(8, dtype=torch.bfloat16)}, tmp_path / "m1.safetensors",
              metadata={"format": "pt", "rank": "8"})
    save_file({"c": torch.zeros(3, dtype=torch.int64)}, tmp_path / "m2.safetensors")
    (tmp_path / "._m3.safetensors").write_bytes(b"junk")
    m = wm.CheckpointMeta.from_dir(tmp_path)
    assert set(m.keys()) == {"a.weight", "b.bias", "c"} and m.metadata["rank"] == "8"
    assert m.tensors["a.weight"] == wm.TensorMeta("F32", (4, 8), 128) and m.total_bytes() == 128 + 16 + 24
    assert wm.safetensors_path_bytes(tmp_path) == 168 and wm.safetensors_path_bytes(tmp_path / "nope") == 0
    keys = ["transformer.blocks.0.attn.to_q.lora_A.weight", "transformer.blocks.0.attn.to_q.lora_B.weight"]
    assert wm.detect_lora_prefix(keys) == "transformer." and wm.detect_lora_prefix(["x.y"]) is None
    assert not wm.keys_contain_lokr(keys) and wm.keys_contain_lokr(["m.lokr_w1"]) and wm.keys_contain_loha(["m.hada_w1_a"])
    assert wm.keys_are_kohya(["lora_unet_double_blocks_0_img_attn_qkv.lora_down.weight"])
    assert wm.parse_rank_alpha("16", "8") == (16.0, 8.0) and wm.parse_rank_alpha("0", None) == (1.0, 1.0)
    assert wm.parse_rank_alpha("x", "4") == (1.0, 4.0) and wm.parse_rank_alpha(None, None) == (1.0, 1.0)
    assert wm.split_factor_key(keys[0], [".lora_A.weight", ".lora_B.weight"]) == ("transformer.blocks.0.attn.to_q",
                                                                                "lora_A.weight")
    table = wm.kohya_table(["double_blocks.0.img_attn.qkv", "single_blocks.3.linear1"])
    assert wm.resolve_kohya_stem("lora_unet_double_blocks_0_img_attn_qkv", table) == "double_blocks.0.img_attn.qkv"
    assert wm.resolve_kohya_stem("lora_unet_missing", table) is None
    assert wm.is_lokr_network_type(" LoKr ") and not wm.is_lokr_network_type(None)


def test_weight_licenses():
    assert lic.FLUX1_SCHNELL.is_well_formed() and lic.FLUX1_SCHNELL.is_permissive()
    assert lic.FLUX1_DEV.is_well_formed() and not lic.FLUX1_DEV.is_permissive()
    bad = lic.WeightLicense("CC-BY-NC-4.0", "CC BY-NC 4.0", "https://example.org/m", "someone", False, None)
    assert not bad.is_well_formed()
    man = json.loads(lic.weight_licenses_manifest_json([lic.WeightLicenseEntry("flux1_dev", lic.FLUX1_DEV),
                                                        lic.WeightLicenseEntry("b200-llama", lic.LLAMA3)]))
    assert [r["provider_id"] for r in man["model_weight_licenses"]] == ["b200-llama", "flux1_dev"]
    with pytest.raises(ValueError):
        lic.weight_licenses_manifest_json([lic.WeightLicenseEntry("x", bad)])


@pytest.mark.parametrize("name", ["nearest", "bilinear", "bicubic", "lanczos"])
@pytest.mark.parametrize("size", [(17, 23), (96, 40), (64, 64)])
def test_resize_matches_pillow(name, size):
    PIL = pytest.importorskip("PIL.Image")
    rng = np.random.default_rng(3)
    a = rng.integers(0, 256, (48, 64, 3), dtype=np.uint8)
    img = Image(64, 48, a.tobytes())
    out = imageops.resize(img, size[0], size[1], name)
    ref = PIL.fromarray(a).resize(size, {"nearest": PIL.NEAREST, "bilinear": PIL.BILINEAR, "bicubic": PIL.BICUBIC,
                                         "lanczos": PIL.LANCZOS}[name])
    got = np.frombuffer(out.pixels, np.uint8).reshape(size[1], size[0], 3)
    assert np.array_equal(got, np.asarray(ref)), np.abs(got.astype(int) - np.asarray(ref).astype(int)).max()


def test_crop_and_mask():
    a = np.zeros((4, 6, 3), np.uint8)
    a[1:3, 2:4] = 255
    img = Image(6, 4, a.tobytes())
    c = imageops.center_crop(img, 2, 2)
    assert c.pixels == bytes([255] * 12)
    assert imageops.mask_from_luma(img).sum() == 4


def test_bs1770_loudness():
    fs = 48000
    t = np.arange(fs * 3) / fs
    sine = 0.5 * np.sin(2 * np.pi * 997 * t)                        # -6.02 dBFS sine
    mono = AudioTrack(fs, 1, sine.astype(np.float32).tolist())
    l1 = audio_dsp.integrated_loudness(mono)
    assert l1 == pytest.approx(-9.03, abs=0.15)                       # 997 Hz mono sine at -6 dBFS peak: -3.01 - 6.02 LUFS
    stereo = AudioTrack(fs, 2, np.stack([sine, sine], 1).reshape(-1).astype(np.float32).tolist())
    assert audio_dsp.integrated_loudness(stereo) == pytest.approx(l1 + 3.01, abs=0.05)
    assert audio_dsp.integrated_loudness(AudioTrack(fs, 1, [0.0] * fs)) == float("-inf")
    norm = audio_dsp.normalize_loudness(mono, -16.0)
    assert audio_dsp.integrated_loudness(norm) == pytest.approx(-16.0, abs=0.1)
    assert audio_dsp.mixdown_mono(stereo).channels == 1 and math.isfinite(audio_dsp.integrated_loudness(norm))


def test_sdxl_ldm_key_remap():
    import torch

    from inference_b200.contracts.gen_core.sdxl_ldm import SdxlComponent as C, apply_remap, remap_sdxl_ldm_key as r

    a = r("model.diffusion_model.input_blocks.7.0.out_layers.3.weight")
    assert (a.op, a.component, a.key) == ("rename", C.UNET, "down_blocks.2.resnets.0.conv2.weight")
    a = r("first_stage_model.decoder.up.1.block.2.nin_shortcut.weight")
    assert (a.op, a.component, a.key) == ("rename", C.VAE, "decoder.up_blocks.2.resnets.2.conv_shortcut.weight")
    a = r("conditioner.embedders.1.model.transformer.resblocks.9.attn.in_proj_weight")
    assert a.op == "split_qkv" and a.keys == tuple(f"text_model.encoder.layers.9.self_attn.{n}_proj.weight" for n in "qkv")
    assert r("model.diffusion_model.time_embed.0.weight").key == "time_embedding.linear_1.weight"
    assert r("model.diffusion_model.input_blocks.0.0.bias").key == "conv_in.bias"
    assert r("model.diffusion_model.input_blocks.3.0.op.weight").key == "down_blocks.0.downsamplers.0.conv.weight"
    assert r("model.diffusion_model.input_blocks.4.1.proj_in.weight").key == "down_blocks.1.attentions.0.proj_in.weight"
    assert r("model.diffusion_model.middle_block.1.norm.weight").key == "mid_block.attentions.0.norm.weight"
    assert r("model.diffusion_model.middle_block.2.in_layers.0.weight").key == "mid_block.resnets.1.norm1.weight"
    assert r("model.diffusion_model.output_blocks.2.2.conv.weight").key == "up_blocks.0.upsamplers.0.conv.weight"
    assert r("model.diffusion_model.output_blocks.5.1.conv.weight").key == "up_blocks.1.upsamplers.0.conv.weight"
    assert r("conditioner.embedders.0.transformer.text_model.final_layer_norm.bias").component is C.CLIP_L
    assert r("conditioner.embedders.1.model.text_projection").op == "transpose"
    assert r("conditioner.embedders.1.model.positional_embedding").key == "text_model.embeddings.position_embedding.weight"
    assert r("conditioner.embedders.1.model.transformer.resblocks.0.mlp.c_fc.bias").key == \
        "text_model.encoder.layers.0.mlp.fc1.bias"
    a = r("first_stage_model.decoder.mid.attn_1.q.weight")
    assert (a.op, a.key) == ("squeeze", "decoder.mid_block.attentions.0.to_q.weight")
    assert r("first_stage_model.encoder.down.2.downsample.conv.bias").key == "encoder.down_blocks.2.downsamplers.0.conv.bias"
    assert r("first_stage_model.decoder.up.3.upsample.conv.weight").key == "decoder.up_blocks.0.upsamplers.0.conv.weight"
    assert r("unrelated.key") is None and r("model.diffusion_model.unknown") is None
    parts = apply_remap({
        "conditioner.embedders.1.model.transformer.resblocks.0.attn.in_proj_bias": torch.arange(6.0),
        "conditioner.embedders.1.model.text_projection": torch.arange(6.0).view(2, 3),
        "first_stage_model.decoder.mid.attn_1.k.weight": torch.zeros(4, 4, 1, 1),
        "model.diffusion_model.out.2.bias": torch.ones(4)})
    g = parts[C.CLIP_BIG_G]
    assert g["text_model.encoder.layers.0.self_attn.k_proj.bias"].tolist() == [2.0, 3.0]
    assert g["text_projection.weight"].shape == (3, 2)
    assert parts[C.VAE]["decoder.mid_block.attentions.0.to_k.weight"].shape == (4, 4)
    assert parts[C.UNET]["conv_out.bias"].shape == (4,)


def test_media_test_tools(tmp_path, monkeypatch):
    import pytest
    import torch

    from inference_b200.contracts.gen_core.media import Image
    from inference_b200.testkit import media_tools as mt

    img = Image(3, 2, bytes(range(18)))
    mt.write_ppm(tmp_path / "a.ppm", img)
    back = mt.read_ppm(tmp_path / "a.ppm")
    assert (back.width, back.height, back.pixels) == (3, 2, img.pixels)
    (tmp_path / "c.ppm").write_bytes(b"P6\n# comment\n1 1\n255\n" + bytes([9, 8, 7]))
    assert mt.read_ppm(tmp_path / "c.ppm").pixels == bytes([9, 8, 7])
    (tmp_path / "bad.ppm").write_bytes(b"P5\n1 1\n255\n\x00")
    with pytest.raises(ValueError):
        mt.read_ppm(tmp_path / "bad.ppm")
    assert mt.mean_abs_diff(img, Image(3, 2, bytes([v + 2 for v in range(18)]))) == 2.0
    assert abs(mt.cosine([1, 0], [1, 0]) - 1) < 1e-12 and abs(mt.cosine([1, 0], [0, 1])) < 1e-12
    assert mt.cosine([0, 0], [1, 1]) == 0.0
    assert abs(mt.tensor_cosine(torch.tensor([1.0, 2.0]), torch.tensor([2.0, 4.0])) - 1) < 1e-12
    monkeypatch.setenv("SWB_TEST_DIR", str(tmp_path))
    assert mt.env_path("SWB_TEST_DIR") == tmp_path and mt.env_path_opt("SWB_UNSET_DIR") is None
    with pytest.raises(RuntimeError, match="SWB_UNSET_DIR"):
        mt.env_path("SWB_UNSET_DIR")
    readings = iter([100, 100, 900, 400, 2500, 300, 300, 300, 300, 300, 300, 300])
    probe = lambda: next(readings, 300)
    vp = mt.VramProbe(probe, interval_s=0.001).assert_idle(1.0)
    ph = vp.phase()
    __import__("time").sleep(0.05)
    vp.end_load(ph)
    rep = vp.report().assert_trustworthy(1.0)
    assert rep.baseline_mib == 100 and rep.load_peak_mib == 2500 and abs(rep.load_delta_gb - 2400 / 1024) < 1e-9
    with pytest.raises(AssertionError):
        mt.VramProbe(lambda: 5000).assert_idle(1.0)
    assert mt.cuda_mempool_used_high_bytes() is None or mt.cuda_mempool_used_high_bytes() >= 0


def test_memory_adaptation_ladder():
    from inference_b200.contracts.gen_core.mempolicy import LaneLevers, Lever, StagePeaks, plan_memory_adaptation
    from inference_b200.contracts.gen_core.runtime import OffloadPolicy

    def peaks_at(scale, tileable=True):
        area = scale * scale
        return StagePeaks(9.0 + 11.0 * area, 1.0 + 30.0 * area, (1.0 + 4.0 * area) if tileable else None)
    levers = LaneLevers(8.0, True, 4.6, (0.75, 0.5))
    plan = plan_memory_adaptation(100.0, levers, peaks_at)
    assert plan.engaged == [] and plan.residency is OffloadPolicy.RESIDENT and plan.feasible and plan.resolution_scale == 1.0
    plan = plan_memory_adaptation(12.0, levers, peaks_at)
    assert plan.engaged == sorted(plan.engaged)
    plan = plan_memory_adaptation(32.0, levers, peaks_at)
    assert plan.engaged == [Lever.SEQUENTIAL_RESIDENCY] and plan.residency is OffloadPolicy.SEQUENTIAL
    assert not plan.tile_decode and not plan.quantize_branch and plan.feasible and plan.projected_peak_gib <= 32.0
    plan = plan_memory_adaptation(22.0, levers, peaks_at)
    assert plan.engaged == [Lever.SEQUENTIAL_RESIDENCY, Lever.VAE_DECODE_TILING] and not plan.quantize_branch
    plan = plan_memory_adaptation(16.0, levers, peaks_at)
    assert plan.quantize_branch and plan.resolution_scale == 1.0 and Lever.RESOLUTION_REDUCTION not in plan.engaged
    plan = plan_memory_adaptation(13.0, levers, peaks_at)
    assert Lever.RESOLUTION_REDUCTION in plan.engaged and plan.resolution_scale == 0.75 and plan.feasible
    assert plan.residency is OffloadPolicy.SEQUENTIAL and plan.quantize_branch
    assert plan_memory_adaptation(8.0, levers, peaks_at).resolution_scale == 0.5
    plan = plan_memory_adaptation(1.5, levers, peaks_at)
    assert not plan.feasible and plan.projected_peak_gib > 1.5
    bare = LaneLevers(0.0, False, 0.0, ())
    fixed = lambda s: StagePeaks(20.0, 10.0, None)
    ok, no = plan_memory_adaptation(25.0, bare, fixed), plan_memory_adaptation(15.0, bare, fixed)
    assert ok.engaged == [] and ok.feasible and not no.feasible and no.engaged == []
    unwired = LaneLevers(8.0, False, 4.6, (0.75, 0.5))
    plan = plan_memory_adaptation(35.0, unwired, peaks_at)
    assert Lever.SEQUENTIAL_RESIDENCY not in plan.engaged and plan.residency is OffloadPolicy.RESIDENT
    assert plan.tile_decode and plan.feasible


def test_media_text_tokenizer_templates_truncation_and_padding():
    from inference_b200.contracts.gen_core.tokenizer import PromptTemplate as P, TextTokenizer, TokenizerConfig
    from inference_b200.testkit.synthetic import wordlevel_tokenizer_json

    assert P.NONE.render("x") == "x"
    assert P.QWEN_INSTRUCT.render("a cat") == "<|im_start|>user\na cat<|im_end|>\n<|im_start|>assistant\n"
    assert P.QWEN_INSTRUCT_NO_THINK.render("p").endswith("<think>\n\n</think>\n\n")
    assert P.QWEN_IMAGE.render("p").startswith("<|im_start|>system\nDescribe the image by detailing the color")
    assert P.FLUX2_DEV_MISTRAL.render("p").startswith("[SYSTEM_PROMPT]You are an AI") and \
        P.FLUX2_DEV_MISTRAL.render("p").endswith("[/SYSTEM_PROMPT][INST]p[/INST]")
    js = wordlevel_tokenizer_json(64)
    t = TextTokenizer.from_json_str(js, TokenizerConfig(max_length=4, pad_token_id=0))
    out = t.tokenize("the cat sat on mat")
    assert len(out.ids) == 4 and out.mask == [1, 1, 1, 1]                  # right truncation
    assert t.tokenize("").ids == [] and t.decode(out.ids[:2]) == "the cat"
    p = TextTokenizer.from_json_str(js, TokenizerConfig(max_length=6, pad_token_id=7, pad_to_max_length=True))
    out = p.tokenize("hello world")
    assert out.ids[2:] == [7] * 4 and out.mask == [1, 1, 0, 0, 0, 0]
    assert p.tokenize("").mask == [0] * 6                                   # an empty prompt still pads
    assert p.encode_ids("hello world", False) == out.ids[:2] == p.encode_chat_ids("hello world", False)
    assert p.config().max_length == 6 and len(p.constraint_decode_table().pieces) == 64
