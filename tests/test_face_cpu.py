"""Face stack: host geometry against the properties the reference's tests state (similarity recovery, lossless
identity warp and resize, constant preservation, suppression order), detection decoding on hand-made network outputs,
and the detector / embedder networks end to end on random weights of the real topology."""
import math

import numpy as np
import pytest
import torch

from inference_b200.contracts.errors import InferenceError
from inference_b200.contracts.gen_core.media import Image
from inference_b200.contracts.gen_core.traits import FaceDetection
from inference_b200.media import face as Fc


def test_umeyama_recovers_a_known_similarity():
    s, ct, st, tx, ty = 1.7, 0.8, 0.6, 12.0, -5.0
    src = np.array([[s * (ct * x - st * y) + tx, s * (st * x + ct * y) + ty] for x, y in Fc.ARCFACE_DST])
    m = Fc.umeyama(src, Fc.ARCFACE_DST)
    want = np.array([[ct / s, st / s, -(ct * tx + st * ty) / s], [-st / s, ct / s, (st * tx - ct * ty) / s]])
    assert np.allclose(m, want, atol=1e-9)
    assert np.allclose(Fc.invert_affine(Fc.invert_affine(m)), m, atol=1e-12)


def test_fixed_point_warp_and_resize():
    src = (np.arange(8 * 8 * 3) % 251).astype(np.uint8)
    ident = np.array([[1.0, 0, 0], [0, 1.0, 0]])
    assert np.array_equal(Fc.warp_affine(src, 8, 8, ident, 8, 8).reshape(-1), src)
    shifted = Fc.warp_affine(src, 8, 8, np.array([[1.0, 0, 2.0], [0, 1.0, 0]]), 8, 8, border=(9, 9, 9)).reshape(8, 8, 3)
    assert np.array_equal(shifted[:, 2:], src.reshape(8, 8, 3)[:, :6]) and (shifted[:, :2] == 9).all()
    assert np.array_equal(Fc.resize_bilinear_cv2(src, 8, 8, 8, 8).reshape(-1), src)
    const = np.full(40 * 10 * 3, 77, dtype=np.uint8)
    assert (Fc.resize_bilinear_cv2(const, 40, 10, 13, 7) == 77).all()
    up = Fc.resize_bilinear_cv2(np.array([0, 0, 0, 100, 100, 100], dtype=np.uint8), 1, 2, 1, 4)[0, :, 0]
    assert up.tolist() == [0, 25, 75, 100]                                  # half-pixel centres, OpenCV convention
    with pytest.raises(InferenceError):
        Fc.warp_affine(src[:-1], 8, 8, ident, 8, 8)
    with pytest.raises(InferenceError):
        Fc.resize_bilinear_cv2(src, 8, 8, 0, 4)
    blob, scale = Fc.detector_blob(np.zeros(100 * 200 * 3, dtype=np.uint8), 100, 200)
    assert blob.shape == (1, 3, 640, 640) and scale == 3.2 and abs(blob[0, 0, 0, 0].item() + 127.5 / 128) < 1e-6
    with pytest.raises(InferenceError):
        Fc.detector_blob(np.zeros(1 * 2000 * 3, dtype=np.uint8), 1, 2000)


def test_suppression_and_decoding():
    det = lambda s, x: FaceDetection((x, 0.0, x + 10.0, 10.0), [(0.0, 0.0)] * 5, s)      # noqa: E731
    kept = Fc.nms([det(0.5, 0.0), det(0.9, 200.0), det(0.7, 300.0), det(0.8, 2.0)], 0.4)
    assert [d.score for d in kept] == [0.9, 0.8, 0.7]                       # 0.5 overlaps the 0.8 box
    # one firing anchor on stride 16: cell (row 3, col 5), second anchor
    s_w, a = Fc.random_face_weights(0, 4)
    det_net = Fc.Scrfd(s_w, "cpu")
    n16 = (640 // 16) ** 2 * 2
    scores = torch.zeros(n16, 1)
    r = (3 * 40 + 5) * 2 + 1
    scores[r] = 0.9
    bbox, kps = torch.zeros(n16, 4), torch.zeros(n16, 10)
    bbox[r] = torch.tensor([1.0, 2.0, 3.0, 4.0])
    kps[r] = torch.arange(10.0) * 0.5
    empty = lambda s: (s, torch.zeros((640 // s) ** 2 * 2, 1), torch.zeros((640 // s) ** 2 * 2, 4), torch.zeros((640 // s) ** 2 * 2, 10))      # noqa: E731
    det_net._forward = lambda x: [empty(8), (16, scores, bbox, kps), empty(32)]
    (d,) = det_net.detect(torch.zeros(1, 3, 640, 640), det_scale=2.0)
    cx, cy = 5 * 16, 3 * 16
    assert d.bbox == ((cx - 16) / 2, (cy - 32) / 2, (cx + 48) / 2, (cy + 64) / 2) and abs(d.score - 0.9) < 1e-6
    assert d.landmarks[1] == ((cx + 1.0 * 16) / 2, (cy + 1.5 * 16) / 2)


def test_networks_end_to_end_on_random_weights():
    s_w, a_w = Fc.random_face_weights(1, 4)
    fa = Fc.FaceAnalysis(Fc.Scrfd(s_w, "cpu"), Fc.ArcFace(a_w, "cpu"))
    outs = fa.scrfd._forward(torch.randn(1, 3, 640, 640))
    assert [(s, sc.shape[0]) for s, sc, _, _ in outs] == [(8, 12800), (16, 3200), (32, 800)]
    x = torch.randn(2, 3, 112, 112)
    e = fa.arcface.forward(x)
    assert e.shape == (2, 512) and torch.allclose(fa.arcface.forward(x[1:]), e[1:], rtol=1e-3, atol=1e-2 * e.abs().max().item())
    g = np.random.default_rng(0)
    img = Image(96, 64, g.integers(0, 255, 64 * 96 * 3, dtype=np.uint8).tobytes())
    blob, _ = Fc.detector_blob(img.pixels, img.height, img.width)
    all_scores = torch.cat([sc[:, 0] for _, sc, _, _ in fa.scrfd._forward(blob)])
    fa.det_thresh = float(all_scores.topk(12).values[-1])                   # random weights: keep the dozen best cells
    faces = fa.analyze(img)
    assert faces and all(len(f.embedding) == 512 and len(f.landmarks) == 5 for f in faces)
    areas = [max(f.bbox[2] - f.bbox[0], 0.0) * max(f.bbox[3] - f.bbox[1], 0.0) for f in faces]
    assert all(a >= b - 1e-3 for a, b in zip(areas, areas[1:]))
    assert fa.largest_face(img).embedding == faces[0].embedding
    assert fa.descriptor().id == "insightface_antelopev2" and fa.detect(img)[0].embedding is None
    fa.det_thresh = 2.0
    with pytest.raises(InferenceError):
        fa.largest_face(img)
