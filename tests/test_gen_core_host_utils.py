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
