"""Qwen3-VL pieces against Hugging Face transformers on a random tiny configuration: vision tower output and DeepStack
taps, image -> patch layout, three-axis position ids, the interleaved M-RoPE table, and the whole multimodal forward
(embedding splice + DeepStack injection) through the oracle decoder."""
import pytest
import torch

from inference_b200.models import qwen3_vl as V

transformers = pytest.importorskip("transformers")


def _hf(seed=0):
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    cfg = Qwen3VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, vocab_size=200, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True}, tie_word_embeddings=False),
        vision_config=dict(depth=4, hidden_size=48, num_heads=4, intermediate_size=96, patch_size=4, temporal_patch_size=2,
                           spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1, 2]),
        image_token_id=150, video_token_id=151, vision_start_token_id=152, vision_end_token_id=153)
    torch.manual_seed(seed)
    return cfg, Qwen3VLForConditionalGeneration(cfg).eval()


def test_vision_tower_matches_hugging_face():
    cfg, model = _hf()
    vc = V.Qwen3VlVisionConfig.from_json(cfg.to_dict())
    assert (vc.depth, vc.hidden_size, vc.patch_dim, vc.grid_side) == (4, 48, 96, 6)
    tower = V.Qwen3VlVisionTower(vc, dict(model.state_dict()))
    g = torch.Generator().manual_seed(1)
    grids = [(1, 4, 6), (1, 2, 2)]
    patches = torch.randn(4 * 6 + 2 * 2, vc.patch_dim, generator=g)
    with torch.no_grad():
        ref = model.model.visual(patches, grid_thw=torch.tensor(grids))
    out, taps = tower.forward(patches, grids)
    assert out.shape == (7, 64) and len(taps) == 3
    torch.testing.assert_close(out, ref.pooler_output, atol=2e-5, rtol=1e-4)
    for a, b in zip(taps, ref.deepstack_features):
        torch.testing.assert_close(a, b, atol=2e-5, rtol=1e-4)


def test_patch_layout_and_smart_resize():
    vc = V.Qwen3VlVisionConfig(patch_size=4, hidden_size=48, num_heads=4)
    assert V.smart_resize(100, 37, 8, min_pixels=64, max_pixels=10 ** 6) == (96, 40)          # round-half-even, as Python rounds 12.5
    assert V.smart_resize(1000, 1000, 32, max_pixels=256 * 256)[0] <= 256
    img = torch.arange(16 * 24 * 3, dtype=torch.float32).remainder(251).view(16, 24, 3).to(torch.uint8)
    patches, grid = V.image_to_patches(img, vc, min_pixels=16, max_pixels=10 ** 6)
    assert grid == (1, 4, 6) and patches.shape == (24, 3 * 2 * 4 * 4)
    # merge order: patch 1 is (row 0, col 1), patch 2 is (row 1, col 0); channel-major, frame repeated
    norm = (img.float() / 255 - 0.5) / 0.5
    p2 = patches[2].view(3, 2, 4, 4)
    torch.testing.assert_close(p2[:, 0], norm[4:8, 0:4].permute(2, 0, 1))
    torch.testing.assert_close(p2[:, 1], p2[:, 0])
    torch.testing.assert_close(patches[4].view(3, 2, 4, 4)[:, 0], norm[0:4, 8:12].permute(2, 0, 1))


def test_position_ids_and_interleaved_table_match_hugging_face():
    cfg, model = _hf()
    ids = [5, 6, 152] + [150] * 6 + [153, 7, 8, 152] + [150] * 1 + [153, 9]
    grids = [(1, 4, 6), (1, 2, 2)]
    pos, nxt = V.mrope_positions(ids, grids, 150)
    mm = torch.zeros(1, len(ids), dtype=torch.int32)
    mm[0, [i for i, t in enumerate(ids) if t == 150]] = 1
    ref, delta = model.model.get_rope_index(torch.tensor([ids]), mm_token_type_ids=mm, image_grid_thw=torch.tensor(grids))
    assert torch.equal(pos, ref[:, 0]) and nxt == int(ref.max()) + 1 and int(delta) == nxt - len(ids)
    rot = model.model.language_model.rotary_emb
    cos_ref, sin_ref = rot(torch.zeros(1, 1, 32), ref)
    cos, sin = V.interleaved_mrope_table(pos, rot.inv_freq, (6, 5, 5))
    torch.testing.assert_close(cos, cos_ref[0, :, :16], atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(sin, sin_ref[0, :, :16], atol=1e-6, rtol=1e-6)
