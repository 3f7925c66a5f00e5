"""Media-engine commons on the CPU: video tiling policy and blend driver, weight map, memory probe parsing,
budgeted attention, cache slot."""
import math
import os

import pytest
import torch

from inference_b200.contracts.gen_core import video_tiling as vt


def test_trapezoid_and_splits():
    assert vt.trapezoidal_mask(4, 0, 0, False) == [1.0] * 4
    m = vt.trapezoidal_mask(5, 0, 2, False)
    assert m[0] == 1.0 and m[2] == 1.0 and abs(m[3] - 2 / 3) < 1e-6 and abs(m[4] - 1 / 3) < 1e-6
    m = vt.trapezoidal_mask(5, 2, 0, True)
    assert abs(m[0]) < 1e-6 and abs(m[1] - 0.5) < 1e-6 and m[2] == 1.0
    assert vt.split_spatial(2, 1, 4) == ([0, 1, 2], [2, 3, 4], [0, 1, 1], [1, 1, 0])
    starts, _, left, _ = vt.split_temporal(2, 1, 3)
    assert starts == [0, 0] and left == [0, 2]
    for size, overlap in [(8, 8), (8, 16), (0, 0), (0, 4)]:
        s, e, l, r = vt.split_spatial(size, overlap, 64)
        assert s and len(s) == len(e) and len(l) == len(r) and e[-1] == 64


def test_needs_tiling_and_plan_dims():
    C = vt.VideoTilingConfig
    cfg = C.spatial_only(64, 32)
    assert cfg.needs_tiling(vt.LTX, 1, 4, 4) and not cfg.needs_tiling(vt.LTX, 10, 2, 2)
    assert cfg.needs_tiling(vt.WAN, 1, 9, 4) and not cfg.needs_tiling(vt.WAN, 10, 8, 8)
    tc = C.temporal_only(16, 8)
    assert tc.needs_tiling(vt.LTX, 3, 2, 2) and not tc.needs_tiling(vt.LTX, 2, 99, 99)
    assert tc.needs_tiling(vt.WAN, 5, 2, 2) and not tc.needs_tiling(vt.WAN, 4, 99, 99)
    p = tc.plan(vt.LTX, 3, 2, 2)
    assert (p.out_f, p.out_h, p.out_w, p.t[0].out_start) == (17, 64, 64, 0)
    p = tc.plan(vt.WAN, 6, 2, 2)
    assert (p.out_f, p.out_h, p.out_w, p.t[0].out_start, p.t[-1].out_stop) == (24, 16, 16, 0, 24)
    assert C.auto(512, 512, 33) is None
    assert C.auto(1024, 1024, 33).spatial.tile_px == 512 and C.auto(1280, 720, 33).spatial.tile_px == 384
    assert C.auto(512, 512, 120).temporal == vt.TemporalTiling(48, 16)
    assert C.auto(1280, 1280, 120) == C.aggressive()


@pytest.mark.parametrize("vae,f,h,w", [(vt.WAN, 9, 9, 13), (vt.WAN22, 9, 9, 13), (vt.LTX, 5, 5, 5)])
def test_plan_covers_every_output_position(vae, f, h, w):
    cfg = vt.VideoTilingConfig(vt.SpatialTiling(4 * vae.spatial_scale, 2 * vae.spatial_scale),
                               vt.TemporalTiling(3 * vae.temporal_scale, vae.temporal_scale))
    plan = cfg.plan(vae, f, h, w)
    for tiles, out in ((plan.t, plan.out_f), (plan.h, plan.out_h), (plan.w, plan.out_w)):
        weight = [0.0] * out
        for t in tiles:
            for i, m in enumerate(t.mask):
                weight[t.out_start + i] += m
        assert all(v > 1e-6 for v in weight)
    plan = vt.VideoTilingConfig.spatial_only(64, 64).plan(vt.WAN, 1, 16, 16)       # tile == overlap
    for tiles, out in ((plan.h, plan.out_h), (plan.w, plan.out_w)):
        weight = [0.0] * out
        for t in tiles:
            for i, m in enumerate(t.mask):
                weight[t.out_start + i] += m
        assert all(v > 1e-6 for v in weight)


def _lin_cost(accum, tile):
    return lambda of, oh, ow, tf, th, tw: accum * (of * oh * ow) + tile * (tf * th * tw)


CANDS = vt.TileCandidates((256, 192, 128), 64, ((32, 8), (16, 4)))


def test_budgeted_plan():
    cost = _lin_cost(4e-8, 4e-6)
    assert vt.budgeted_plan(vt.WAN, 512, 512, 64, 1000.0, CANDS, cost) is None
    assert vt.WAN.writable_frame_cap(720, 1280) == 24 and vt.LTX.writable_frame_cap(720, 1280) == 291
    assert vt.WAN.with_channels(48).writable_frame_cap(720, 1280) == 48
    free = lambda *a: 0.0
    assert vt.budgeted_plan(vt.WAN, 720, 1280, 24, math.inf, CANDS, free) is None
    past = vt.budgeted_plan(vt.WAN, 720, 1280, 25, math.inf, CANDS, free)
    assert past is not None and past.temporal is not None and past.temporal.tile_frames <= 24
    single = cost(64, 512, 512, 64, 512, 512)
    assert single > 20.0
    cfg = vt.budgeted_plan(vt.WAN, 512, 512, 64, 20.0, CANDS, cost)
    th = min(cfg.spatial.tile_px, 512) if cfg.spatial else 512
    tf = min(cfg.temporal.tile_frames, 64) if cfg.temporal else 64
    assert cost(64, 512, 512, tf, th, th) <= 20.0 < single
    with pytest.raises(vt.TilingBudgetError) as e:
        vt.budgeted_plan(vt.WAN, 4096, 4096, 257, 0.001, CANDS, cost)
    assert e.value.kind == "accumulators"


def test_decode_tiled_blend_and_budget_helpers(monkeypatch):
    from inference_b200.media import vae_tiling as drv

    def upsample_wan(tile):
        b, _, f, h, w = tile.shape
        return torch.full((b, 3, f * 4, h * 8, w * 8), float(tile.flatten()[0]))

    cfg = vt.VideoTilingConfig.spatial_only(64, 16)
    out = drv.decode_tiled(vt.WAN, "t", torch.full((1, 4, 1, 16, 16), 0.7), cfg, upsample_wan)
    assert out.shape == (1, 3, 4, 128, 128) and (out - 0.7).abs().max() < 1e-4
    out = drv.decode_tiled(vt.WAN, "t", torch.full((1, 4, 2, 8, 8), 0.5), cfg, upsample_wan)
    assert out.shape == (1, 3, 8, 64, 64)
    # a position-dependent decoder: tiled decode of a per-pixel map equals the single pass
    lat = torch.randn(1, 1, 1, 24, 20)
    up = lambda t: t.repeat_interleave(8, 3).repeat_interleave(8, 4).repeat_interleave(4, 2).expand(-1, 3, -1, -1, -1)
    torch.testing.assert_close(drv.decode_tiled(vt.WAN, "t", lat, cfg, up), up(lat), atol=1e-5, rtol=1e-5)

    monkeypatch.setenv("SWB_TEST_VAE_BUDGET_GIB", "42.5")
    assert drv.safe_budget_gib("SWB_TEST_VAE_BUDGET_GIB", 0.85, 16.0) == 42.5
    monkeypatch.delenv("SWB_TEST_VAE_BUDGET_GIB")
    assert drv.safe_budget_gib("SWB_TEST_VAE_BUDGET_GIB", 0.85, 16.0, total_probe=lambda: None) == 16.0
    assert drv.safe_budget_gib("SWB_TEST_VAE_BUDGET_GIB", 0.5, 16.0, total_probe=lambda: 180.0) == 90.0
    assert drv.free_aware_budget_gib(-5.0, 0.85) == 0.0
    assert abs(drv.free_aware_safe_budget_gib("SWB_UNSET", 0.85, 16.0, free_probe=lambda: 66.0) - 66 * 0.85) < 1e-9
    assert drv.free_aware_safe_budget_gib("SWB_UNSET", 0.85, 16.0, free_probe=lambda: None) == 16.0
    cost = lambda of, oh, ow, tf, th, tw: (10.0 * of * oh * ow + 1000.0 * th * tw) / 2 ** 30
    cands = vt.TileCandidates((512, 256, 128), 32, ())
    narrow = vt.WAN.with_channels(1)
    assert drv.plan_tiling("t", narrow, 1024, 1024, 49, 1e6, cands, cost) is None
    some = drv.plan_tiling("t", narrow, 1024, 1024, 49, 1.0, cands, cost)
    assert some.spatial is not None and some.temporal is None
    with pytest.raises(Exception, match="Reduce the resolution"):
        drv.plan_tiling("t", narrow, 4096, 4096, 257, 0.001, cands, cost)


def test_weights_map(tmp_path):
    from inference_b200.contracts.errors import LoadError
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media.weights import Weights

    a, b = tmp_path / "model-00001-of-00002.safetensors", tmp_path / "model-00002-of-00002.safetensors"
    save_file({"a.weight": torch.tensor([1.0]), "idx": torch.tensor([3], dtype=torch.int32)}, a)
    save_file({"b.weight": torch.tensor([2.0]), "te.x": torch.tensor([5.0])}, b)
    w = Weights.from_files([a, b], "cpu", torch.bfloat16)
    assert w.require("a.weight").dtype == torch.bfloat16 and w.require("idx").dtype == torch.int32
    assert float(w.require("b.weight")) == 2.0 and w.contains("te.x") and len(w) == 4
    assert sorted(Weights.from_files([a, b], prefixes=["te.", "a."]).keys()) == ["a.weight", "te.x"]
    assert list(w.with_prefix("te.").keys()) == ["x"]
    with pytest.raises(LoadError, match="missing tensor: nope"):
        w.require("nope")
    dup = tmp_path / "dup.safetensors"
    save_file({"a.weight": torch.tensor([9.0])}, dup)
    with pytest.raises(LoadError, match="duplicate tensor key 'a.weight'"):
        Weights.from_files([a, dup])


def test_gpu_probe_parsing():
    from inference_b200.media import gpu_probe as gp

    for p in gp.candidate_paths():
        assert p.is_absolute() and p.name.startswith("nvidia-smi")
    assert gp.first_existing([gp.Path("/nope/a/nvidia-smi"), gp.Path(os.__file__)]) == gp.Path(os.__file__)
    assert gp.first_existing([gp.Path("/nope/a/nvidia-smi")]) is None
    assert abs(gp.parse_min_mib_line_gib("24576\n49152\n") - 24.0) < 1e-9
    assert gp.parse_min_mib_line_gib("") is None and gp.parse_min_mib_line_gib("no gpus\n\n") is None
    assert gp.parse_min_mib_line_gib("0\n") is None
    po = gp.parse_rendered_ordinal
    assert (po(None), po("1"), po("2,3"), po(" 1 "), po(""), po("GPU-1a2b"), po("MIG-abc")) == (0, 1, 2, 1, None, None, None)
    calls = []

    def fake(args):
        calls.append(args)
        return "1000\n" if "-i" in args else "183359\n90000\n"
    assert abs(gp.nvidia_smi_min_total_gib(fake) - 90000 / 1024) < 1e-9
    assert abs(gp.nvidia_smi_rendered_free_gib(fake, {"CUDA_VISIBLE_DEVICES": "3"}) - 1000 / 1024) < 1e-9
    assert calls[-1][-2:] == ["-i", "3"]
    assert abs(gp.nvidia_smi_rendered_free_gib(fake, {"CUDA_VISIBLE_DEVICES": "GPU-x"}) - 90000 / 1024) < 1e-9
    assert gp.nvidia_smi_min_free_gib(lambda a: None) is None


def test_budgeted_attention_and_cache_slot():
    from inference_b200.media.attention_budget import ATTN_SCORES_BUDGET as B, query_block, sdpa_budgeted_bhsd, \
        sdpa_budgeted_flat
    from inference_b200.utils.sync import Slot, cached

    assert query_block(2 * 10 * 16384, 16384, B) < 16384 and query_block(65536, 65536, B) < 65536
    assert query_block(32 * 8192, 8200, B) < 8200
    assert query_block(20 * 4096, 4096, B) == 4096 and query_block(16384, 16384, B) == 16384
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(3, 7, 4, generator=g) for _ in range(3))
    single = sdpa_budgeted_flat(q, k, v, 0.5, 2 ** 62)
    torch.testing.assert_close(single, sdpa_budgeted_flat(q, k, v, 0.5, 1))
    torch.testing.assert_close(single, sdpa_budgeted_flat(q, k, v, 0.5, 63))
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.5)
    torch.testing.assert_close(single, ref)
    mask = torch.randn(1, 1, 7, 7, generator=g)
    a = sdpa_budgeted_bhsd(q[None], k[None], v[None], 0.5, mask, 2 ** 62)
    torch.testing.assert_close(a, sdpa_budgeted_bhsd(q[None], k[None], v[None], 0.5, mask, 40))
    slot, n = Slot(), []
    def load():
        n.append(1)
        if len(n) == 1:
            raise RuntimeError("first load fails")
        return "value"
    with pytest.raises(RuntimeError):
        cached(slot, load)
    assert cached(slot, load) == "value" and cached(slot, load) == "value" and len(n) == 2
