"""PuLID-FLUX: the EVA tower's rotary tables and pair rotation, the antialiased bicubic transform against Pillow, the
face parser's pieces, the IDFormer / cross-attention schedule, the DiT hook seam, and one identity-steered render on
synthetic checkpoints."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from inference_b200.contracts.errors import InferenceError
from inference_b200.contracts.gen_core.media import Image
from inference_b200.media import face as Fc
from inference_b200.media import pulid as P


def test_eva_rotary_tables_and_pair_rotation():
    assert P.rotate_pairs(torch.tensor([1.0, 2.0, 3.0, 4.0])).tolist() == [-2.0, 1.0, -4.0, 3.0]
    cos, sin = P.eva_rope_tables(64, 24, 16, 10000.0)
    assert cos.shape == (576, 64)
    assert torch.allclose(cos[0], torch.ones(64)) and torch.allclose(sin[0], torch.zeros(64))
    # token (row 3, column 5): first half follows the row, second the column; adjacent lanes share a frequency
    tok = 3 * 24 + 5
    f1 = 1.0 / 10000.0 ** (2.0 / 32)
    assert cos[tok, 0] == pytest.approx(np.cos(3 / 24 * 16), abs=1e-6) and cos[tok, 1] == cos[tok, 0]
    assert cos[tok, 2] == pytest.approx(np.cos(3 / 24 * 16 * f1), abs=1e-6)
    assert sin[tok, 32] == pytest.approx(np.sin(5 / 24 * 16), abs=1e-6)


def test_transform_matches_pillow_bicubic():
    from PIL import Image as PI

    g = np.random.default_rng(0)
    for (h, w, size) in ((64, 80, 24), (20, 20, 28), (33, 33, 33)):
        a = g.integers(64, 192, (h, w, 3), dtype=np.uint8)          # mid-range: no overshoot for Pillow to clip
        ref = np.asarray(PI.fromarray(a).resize((size, size), PI.BICUBIC)).astype(np.float32) / 255.0
        x = torch.from_numpy(a.astype(np.float32) / 255.0).permute(2, 0, 1)[None]
        got = P.eva_transform(x, size)[0]
        mean, std = torch.tensor(P.EVA_MEAN).view(3, 1, 1), torch.tensor(P.EVA_STD).view(3, 1, 1)
        back = (got * std + mean).permute(1, 2, 0).numpy()
        assert np.abs(back.clip(0, 1) - ref).max() < 1.5 / 255            # Pillow rounds to 8 bits between the passes
    m = P._resize_matrix(17, 9)
    assert np.allclose(m.sum(1), 1.0) and np.allclose(P._resize_matrix(7, 7), np.eye(7))
    with pytest.raises(InferenceError):
        P.eva_transform(torch.zeros(2, 3, 8, 8), 4)


def test_eva_tower_block_against_a_restatement():
    cfg = P.EvaConfig(image_size=28, patch=7, embed_dim=32, depth=6, num_heads=2, proj_dim=12, pt_seq_len=4,
                      hidden_capture=(1, 2, 3, 4, 5), mlp_dim=40)
    w = P.random_eva_weights(cfg, 1)
    tower = P.EvaVisionTower(w, cfg)
    x = torch.randn(1, 3, 28, 28, generator=torch.Generator().manual_seed(2))
    proj, hidden = tower.forward(x)
    assert proj.shape == (1, 12) and len(hidden) == 5 and hidden[0].shape == (1, 17, 32)
    # the second captured state is block 1 applied to the first
    h0, p = hidden[0], "blocks.1"
    ln = lambda t, n: F.layer_norm(t, (t.shape[-1],), w[n + ".weight"], w[n + ".bias"], 1e-6)       # noqa: E731
    cos, sin = P.eva_rope_tables(16, 4, 4, 10000.0)

    def rope(t):                                 # [1, H, N, hd]
        pat = t[:, :, 1:]
        e, o = pat[..., 0::2], pat[..., 1::2]
        c, s = cos[:, 0::2], sin[:, 0::2]
        return torch.cat([t[:, :, :1], torch.stack([e * c - o * s, o * c + e * s], -1).flatten(-2)], 2)

    n1 = ln(h0, p + ".norm1")
    hs = lambda t: t.view(1, 17, 2, 16).transpose(1, 2)                                              # noqa: E731
    q = rope(hs(F.linear(n1, w[p + ".attn.q_proj.weight"], w[p + ".attn.q_bias"])))
    k = rope(hs(F.linear(n1, w[p + ".attn.k_proj.weight"])))
    v = hs(F.linear(n1, w[p + ".attn.v_proj.weight"], w[p + ".attn.v_bias"]))
    a = (torch.softmax(q @ k.transpose(-1, -2) / 4.0, -1) @ v).transpose(1, 2).reshape(1, 17, 32)
    y = h0 + F.linear(ln(a, p + ".attn.inner_attn_ln"), w[p + ".attn.proj.weight"], w[p + ".attn.proj.bias"])
    n2 = ln(y, p + ".norm2")
    gate = F.silu(F.linear(n2, w[p + ".mlp.w1.weight"], w[p + ".mlp.w1.bias"])) * F.linear(n2, w[p + ".mlp.w2.weight"], w[p + ".mlp.w2.bias"])
    y = y + F.linear(ln(gate, p + ".mlp.ffn_ln"), w[p + ".mlp.w3.weight"], w[p + ".mlp.w3.bias"])
    assert torch.allclose(hidden[1], y, atol=1e-5)


def test_face_parser_pieces():
    x = torch.randn(2, 3, 5, 7)
    up = Fc.upsample_bilinear_align_corners(x, 11, 13)
    assert torch.allclose(up, F.interpolate(x, size=(11, 13), mode="bilinear", align_corners=True), atol=1e-5)
    net = Fc.BiSeNet(Fc.random_bisenet_weights(0, 4), "cpu")
    logits = net.parse_logits(torch.randn(1, 3, 64, 64))
    assert logits.shape == (1, 19, 64, 64) and net.parse_mask(torch.randn(1, 3, 64, 64)).shape == (1, 64, 64)
    rgb = torch.tensor([[[[1.0, 0.5]], [[0.0, 0.5]], [[0.0, 0.5]]]])                       # two pixels: red, grey
    out = Fc.face_features_image(rgb, torch.tensor([[[1, 16]]]))
    assert out[0, :, 0, 0].tolist() == pytest.approx([0.299] * 3) and out[0, :, 0, 1].tolist() == [1.0, 1.0, 1.0]
    assert set(Fc.BG_LABELS) == {0, 7, 8, 9, 14, 15, 16, 18}


def _tiny_pulid(hidden=16, num_ca=2):
    icfg = P.IdFormerConfig(dim=16, depth=5, heads=2, dim_head=8, num_id_token=2, num_queries=4, output_dim=24, id_dim=512 + 12, vit_dim=32)
    return icfg, P.random_pulid_weights(icfg, hidden, num_ca, 3)


def test_idformer_and_injection_schedule():
    icfg, w = _tiny_pulid(num_ca=3)
    f = P.IdFormer(w, icfg)
    hidden = [torch.randn(1, 17, 32) for _ in range(5)]
    emb = f.forward(torch.randn(1, 524), hidden)
    assert emb.shape == (1, 4, 24)
    with pytest.raises(InferenceError):
        f.forward(torch.randn(1, 524), hidden[:4])
    # each scale feeds only its own layer: perturbing the last tower state leaves a 4-scale prefix computation unchanged
    w["swb_ca_config"] = torch.tensor([2, 8])
    ca = P.PulidCa(w, emb, 1.0, 2, 5)
    assert (ca.n_double, ca.num_ca) == (1, 3)
    img = torch.randn(1, 9, 16)
    assert ca.after_double(0, img).shape == (1, 9, 16) and ca.after_double(1, img) is None
    assert ca.after_single(0, img) is not None and ca.after_single(1, img) is None and ca.after_single(4, img) is not None
    assert not torch.allclose(ca.after_single(0, img), ca.after_double(0, img))           # module 1 vs module 0
    half = P.PulidCa(w, emb, 0.5, 2, 5)
    assert torch.allclose(half.after_double(0, img), ca.after_double(0, img) * 0.5, atol=1e-6)
    off = P.PulidCa(w, emb, 0.0, 2, 5)
    assert off.after_double(0, img) is None and off.after_single(0, img) is None
    assert P.l2_normalize_rows(torch.tensor([[3.0, 4.0], [0.0, 0.0]])).tolist() == [[0.6000000238418579, 0.800000011920929], [0.0, 0.0]]


def test_request_floor():
    P.reject_below_floor(P.PulidFluxRequest())
    with pytest.raises(InferenceError, match="steps must be >= 1"):
        P.reject_below_floor(P.PulidFluxRequest(steps=0))
    with pytest.raises(InferenceError, match="multiples of 16"):
        P.reject_below_floor(P.PulidFluxRequest(height=1000))
    r = P.PulidFluxRequest()
    assert (r.width, r.height, r.steps, r.guidance, r.id_weight) == (1024, 1024, 25, 4.0, 1.0)


def test_identity_steered_render(tmp_path):
    from inference_b200.io.safetensors_io import save_file
    from inference_b200.media.flux import write_synthetic_snapshot

    flux = write_synthetic_snapshot(tmp_path / "flux")
    s_w, a_w = Fc.random_face_weights(1, 4)
    fd = tmp_path / "face"
    fd.mkdir()
    save_file(s_w, fd / "scrfd.safetensors")
    save_file(a_w, fd / "arcface.safetensors")
    save_file(Fc.random_bisenet_weights(2, 4), fd / Fc.BISENET_FILE)
    ecfg = P.EvaConfig(image_size=28, patch=7, embed_dim=32, depth=6, num_heads=2, proj_dim=12, pt_seq_len=4,
                       hidden_capture=(1, 2, 3, 4, 5), mlp_dim=40)
    ew = P.random_eva_weights(ecfg, 1)
    ew["swb_eva_config"] = torch.tensor([28, 7, 32, 6, 2, 12, 4, 1, 2, 3, 4, 5, 40])
    save_file(ew, tmp_path / "eva.safetensors")
    icfg = P.IdFormerConfig(dim=16, depth=5, heads=2, dim_head=8, num_id_token=2, num_queries=4, output_dim=24, id_dim=524, vit_dim=32)
    pw = P.random_pulid_weights(icfg, 256, 2, 3)                    # 2 double + 2 single blocks -> 1 + 1 modules
    pw["swb_idformer_config"] = torch.tensor([16, 5, 2, 8, 2, 4, 24, 524, 32])
    pw["swb_ca_config"] = torch.tensor([2, 8])
    save_file(pw, tmp_path / "pulid.safetensors")
    paths = P.PulidFluxPaths(flux, tmp_path / "pulid.safetensors", tmp_path / "eva.safetensors", fd)
    p = P.PulidFlux.load(paths, "cpu")
    g = np.random.default_rng(0)
    ref = Image(96, 64, g.integers(0, 255, 64 * 96 * 3, dtype=np.uint8).tobytes())
    blob, _ = Fc.detector_blob(ref.pixels, ref.height, ref.width)
    scores = torch.cat([sc[:, 0] for _, sc, _, _ in p.face.scrfd._forward(blob)])
    p.face.det_thresh = float(scores.topk(12).values[-1])
    emb = p.compute_id_embedding(ref)
    assert emb.shape == (1, 4, 24) and torch.isfinite(emb).all()
    req = P.PulidFluxRequest(prompt="a portrait", width=256, height=256, steps=2, seed=4)
    on = p.generate(req, ref)
    off = p.generate(P.PulidFluxRequest(**{**req.__dict__, "id_weight": 0.0}), ref)
    assert (on.width, on.height) == (256, 256) and on.pixels != off.pixels
    # zero weight is the plain text-to-image render, and the hooks are removed afterwards
    from inference_b200.contracts.gen_core import GenerationRequest

    plain = p.flux.generate(GenerationRequest(prompt="a portrait", width=256, height=256, steps=2, seed=4, guidance=4.0)).images[0]
    assert plain.pixels == off.pixels
    p.face.det_thresh = 2.0
    with pytest.raises(InferenceError, match="no face"):
        p.generate(req, ref)
    with pytest.raises(P.LoadError):
        P.PulidFlux.load(P.PulidFluxPaths(flux, tmp_path / "missing.safetensors", tmp_path / "eva.safetensors", fd), "cpu")
