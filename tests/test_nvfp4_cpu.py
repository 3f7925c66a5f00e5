"""NVFP4 container: the vectorised packer against a scalar restatement of the format rules, the swizzled scale
layout, the outlier metric and the per-layer activation-precision policy."""
import math

import torch

from inference_b200.ops import nvfp4 as nv


def _e4m3_to_f32(b: int) -> float:
    exp, man = (b >> 3) & 0xF, b & 7
    if exp == 0:
        return man * 2.0 ** -9
    return (1.0 + man / 8.0) * 2.0 ** (exp - 7)


def _scalar_e4m3_from(v: float) -> int:
    if math.isnan(v) or v <= 0:
        return 0
    v = min(v, 448.0)
    best, best_d = 0, float("inf")
    for code in range(0x7F):
        d = abs(_e4m3_to_f32(code) - v)
        if d < best_d or (d == best_d and code % 2 == 0):
            best, best_d = code, d
    return best


def _scalar_e2m1_from(v: float) -> int:
    sign = 8 if math.copysign(1.0, v) < 0 else 0
    mag = min(abs(v), 6.0)
    best, best_d = 0, float("inf")
    for i, m in enumerate(nv.E2M1_MAGS):
        d = abs(m - mag)
        if d < best_d or (d == best_d and i % 2 == 0):
            best, best_d = i, d
    return sign | best


def test_code_rounding_matches_scalar_rules():
    f32 = torch.float32
    vals = torch.cat([torch.linspace(-7, 7, 561), torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -2.5, -0.0])])
    got = nv.e2m1_from_f32(vals).tolist()
    assert got == [_scalar_e2m1_from(torch.tensor(v, dtype=f32).item()) for v in vals.tolist()]
    tab = nv.e4m3_table()
    mids = (tab[:-1] + tab[1:]) / 2
    vals = torch.cat([tab, mids, torch.rand(500) * 500, torch.tensor([0.0, -1.0, 1e-5, 449.0, 1e6])])
    got = nv.e4m3_from_f32(vals).tolist()
    assert got == [_scalar_e4m3_from(v) for v in vals.tolist()]
    assert [_e4m3_to_f32(c) for c in range(0x7F)] == tab.tolist()


def test_pack_matches_scalar_packer_and_roundtrips():
    g = torch.Generator().manual_seed(0)
    rows, cols = 130, 72            # ragged: a partial scale atom in both directions and a padded last block
    w = torch.randn(rows, cols, generator=g) * 0.1
    w[3, 5] = 2.0                    # an outlier sets the global scale
    t = nv.Nvfp4Tensor.pack(w)
    assert (t.cols_padded, t.sf_rows, t.sf_cols) == (80, 256, 8)
    assert t.scales.numel() == nv.Nvfp4Tensor.scale_tensor_len(rows, cols)
    f = lambda x: torch.tensor(x, dtype=torch.float32)
    gs = (f(2.0) / f(6.0 * 448.0)).item()
    assert t.global_scale == gs
    for r, blk in [(0, 0), (3, 0), (129, 4), (64, 2), (31, 3)]:
        c0, c1 = blk * 16, min(blk * 16 + 16, cols)
        a = w[r, c0:c1].abs().max()
        sf = _scalar_e4m3_from((a / f(6.0 * gs)).item())
        assert int(t.scales[nv.scale_offset(r, blk, t.sf_rows)]) == sf
        es = (f(_e4m3_to_f32(sf)) * f(gs))
        for c in range(c0, c0 + 16):
            v = w[r, c] if c < cols else f(0.0)
            code = _scalar_e2m1_from((v / es).item()) if es > 0 else 0
            byte = int(t.packed[r, c // 2])
            assert ((byte >> 4) if c % 2 else (byte & 0xF)) == code
    d = t.dequantize()
    assert d.shape == w.shape
    rel = (d - w).norm() / w.norm()
    assert rel < 0.12
    # packing the dequantised tensor again is a fixed point
    t2 = nv.Nvfp4Tensor.pack(d)
    assert torch.equal(t2.dequantize(), d)


def test_scale_offsets_are_a_permutation_of_the_atom_grid():
    sf_rows, nb = 256, 8
    r = torch.arange(sf_rows).unsqueeze(1).expand(sf_rows, nb)
    b = torch.arange(nb).unsqueeze(0).expand(sf_rows, nb)
    off = nv.scale_offset(r, b, sf_rows).flatten()
    assert sorted(off.tolist()) == list(range(sf_rows * nb))
    assert nv.scale_offset(0, 0, 256) == 0 and nv.scale_offset(1, 0, 256) == 16 and nv.scale_offset(32, 0, 256) == 4
    assert nv.scale_offset(128, 0, 256) == 512 and nv.scale_offset(0, 4, 256) == 1024


def test_outlier_metric_and_policy():
    g = torch.Generator().manual_seed(1)
    x = (torch.rand(64, 256, generator=g) * 2 - 1) * 0.3
    s = nv.OutlierSparsity.from_tensor(x)
    assert s.klass() is nv.OutlierClass.BENIGN and s.w4a4_viable() and s.total_blocks == 64 * 16
    y = x.clone()
    y[:, ::16] = 50.0                # an outlier in every block
    s = nv.OutlierSparsity.from_tensor(y)
    assert s.klass() is nv.OutlierClass.DENSE and not s.w4a4_viable() and s.max_crush_ratio > 100
    z = x.clone()
    z[:8, 0] = 50.0                  # 8 of 1024 blocks
    s = nv.OutlierSparsity.from_tensor(z)
    assert s.outlier_blocks == 8 and s.klass() is nv.OutlierClass.SPARSE
    A = nv.ActPrecision
    assert A.for_outlier_layer("transformer_blocks.7.attn1.to_q") is A.W4A4
    assert A.for_outlier_layer("transformer_blocks.7.attn2.to_q") is A.W4A16
    assert A.for_outlier_layer("caption_projection.linear_1") is A.W4A16
    assert A.for_outlier_layer("proj_out.weight") is A.W4A16
    assert A.for_outlier_layer("blocks.3.proj_out") is A.W4A4
    assert A.for_outlier_layer("blocks.0.ff.net.0") is A.W4A16
    assert A.for_outlier_layer("x.cross_attention.to_k") is A.W4A16
    p = nv.Nvfp4Partition.of(["blocks.1.attn1.to_q", "blocks.1.attn2.to_k", "blocks.2.ff"])
    assert (p.n_w4a4, p.n_w4a16) == (2, 1) and abs(p.w4a4_fraction() - 2 / 3) < 1e-12


def test_linear_cpu_matches_dequantised_matmul_and_w4a4_rounds_activations():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(48, 256, generator=g) * 0.05
    b = torch.randn(48, generator=g)
    x = torch.randn(5, 256, generator=g)
    lin = nv.Nvfp4Linear.from_dense(w, b)
    ref = x @ lin.t.dequantize().t() + b
    torch.testing.assert_close(lin(x), ref)
    lin4 = nv.Nvfp4Linear.from_dense(w, b, layer_name="blocks.4.attn1.to_q")
    assert lin4.act_precision is nv.ActPrecision.W4A4
    ref4 = nv.quantize_activations(x) @ lin.t.dequantize().t() + b
    torch.testing.assert_close(lin4(x), ref4)
    assert lin.nvfp4_footprint_bytes() < lin.bf16_footprint_bytes() / 2   # 48 rows pad to a 128-row scale atom
