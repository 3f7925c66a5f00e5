"""Face analysis stack: SCRFD-10g five-point detector, ArcFace (iresnet100) 512-d embedder and the insightface
alignment between them, behind the `FaceEmbedder` contract (parity: candle-gen-face/src/scrfd.rs, iresnet.rs,
align.rs, face.rs, lib.rs).

Weights are safetensors with batch norms folded into the convolutions and convolution kernels stored
[out, kh, kw, in] (the layout the reference's converter writes): `scrfd.safetensors` (`stem.conv{0..2}`,
`stage{1..4}.{b}.{conv1,conv2,downsample}`, `neck.{lateral,fpn}{0..2}`, `neck.{down,pafpn}{0,1}`,
`head{8,16,32}.{stem0..2,cls,reg,kps,scale}`) and `arcface.safetensors` (`stem.{conv,prelu}`,
`layer{1..4}.{b}.{bn1,conv1,prelu,conv2,downsample}`, `bn2`, `fc`, `features`).

Detection: the image is resized (OpenCV's fixed-point bilinear, reproduced exactly) to fit 640 x 640 from the top-left
corner, normalised by (v - 127.5) / 128, scored on strides 8 / 16 / 32 with two anchors per cell, decoded as distances
from the cell origin, kept above 0.5, and suppressed at IoU 0.4. Embedding: a similarity transform (Umeyama) takes the
five landmarks onto the ArcFace template, OpenCV's fixed-point bilinear warp cuts the 112 x 112 crop, and the network
maps (v - 127.5) / 127.5 to 512 numbers. Faces come back largest first.

The networks are plain convolution stacks: they run through the framework's convolution call on either backend (fp32)."""
from __future__ import annotations

import math
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.traits import FaceDetection, FaceEmbedder, SimpleDescriptor

DET_SIZE, NUM_ANCHORS = 640, 2
SCRFD_STAGES, ARCFACE_LAYERS = (3, 4, 2, 3), (3, 13, 30, 3)
ARCFACE_DST = np.array([[38.2946, 51.6963], [73.5318, 51.5014], [56.0252, 71.7366], [41.5493, 92.3655], [70.7299, 92.2041]])
FACEXLIB_DST_512 = np.array([[192.98138, 239.94708], [318.90277, 240.1936], [256.63416, 314.01935], [201.26117, 371.41043],
                             [313.08905, 371.15118]])
FACEXLIB_BORDER_RGB = (132, 133, 135)


# ---- host geometry ------------------------------------------------------------------------------------------------------
def umeyama(src: np.ndarray, dst: np.ndarray) -> np.ndarray:
    """Least-squares similarity (rotation, uniform scale, translation) taking src [n, 2] onto dst [n, 2]: 2 x 3."""
    src, dst = np.asarray(src, dtype=np.float64), np.asarray(dst, dtype=np.float64)
    sm, dm = src.mean(0), dst.mean(0)
    sc, dc = src - sm, dst - dm
    a = dc.T @ sc / len(src)
    var = (sc ** 2).sum() / len(src)
    u, s, vt = np.linalg.svd(a)
    d = np.ones(2)
    if np.linalg.det(a) < 0:
        d[1] = -1.0
    rot = u @ np.diag(d) @ vt
    scale = (s * d).sum() / var if var > 0 else 1.0
    m = scale * rot
    return np.concatenate([m, (dm - m @ sm)[:, None]], axis=1)


def invert_affine(m: np.ndarray) -> np.ndarray:
    det = m[0, 0] * m[1, 1] - m[0, 1] * m[1, 0]
    d = 1.0 / det if det != 0 else 0.0
    a = np.array([[m[1, 1] * d, -m[0, 1] * d], [-m[1, 0] * d, m[0, 0] * d]])
    return np.concatenate([a, (-a @ m[:, 2])[:, None]], axis=1)


def _check(img: np.ndarray | bytes, h: int, w: int, what: str) -> np.ndarray:
    if h <= 0 or w <= 0:
        raise InferenceError(f"{what}: image has a zero dimension ({h}x{w})")
    a = np.frombuffer(img, dtype=np.uint8) if not isinstance(img, np.ndarray) else img.reshape(-1)
    if a.size < h * w * 3:
        raise InferenceError(f"{what}: buffer of {a.size} bytes too small for {h}x{w}x3")
    return a[: h * w * 3].reshape(h, w, 3)


def warp_affine(src, in_h: int, in_w: int, forward: np.ndarray, out_h: int, out_w: int, border=(0, 0, 0)) -> np.ndarray:
    """OpenCV's INTER_LINEAR warpAffine in its fixed-point form (10-bit matrix, 5-bit sub-pixel fractions, 15-bit
    weights), constant border: [out_h, out_w, 3] uint8."""
    img = _check(src, in_h, in_w, "warp_affine").astype(np.int64)
    im = invert_affine(np.asarray(forward, dtype=np.float64))
    AB, INTER = 10, 5
    xs, ys = np.arange(out_w, dtype=np.float64), np.arange(out_h, dtype=np.float64)
    adelta = np.rint(im[0, 0] * xs * 1024).astype(np.int64)
    bdelta = np.rint(im[1, 0] * xs * 1024).astype(np.int64)
    x0 = np.rint((im[0, 1] * ys + im[0, 2]) * 1024).astype(np.int64) + 16
    y0 = np.rint((im[1, 1] * ys + im[1, 2]) * 1024).astype(np.int64) + 16
    xq, yq = (x0[:, None] + adelta[None, :]) >> (AB - INTER), (y0[:, None] + bdelta[None, :]) >> (AB - INTER)
    sx, sy, fx, fy = xq >> INTER, yq >> INTER, xq & 31, yq & 31
    bord = np.asarray(border, dtype=np.int64)

    def sample(px, py):
        ok = (px >= 0) & (px < in_w) & (py >= 0) & (py < in_h)
        v = img[np.clip(py, 0, in_h - 1), np.clip(px, 0, in_w - 1)]
        return np.where(ok[..., None], v, bord)

    w_tl, w_tr = ((32 - fy) * (32 - fx) * 32)[..., None], ((32 - fy) * fx * 32)[..., None]
    w_bl, w_br = (fy * (32 - fx) * 32)[..., None], (fy * fx * 32)[..., None]
    acc = sample(sx, sy) * w_tl + sample(sx + 1, sy) * w_tr + sample(sx, sy + 1) * w_bl + sample(sx + 1, sy + 1) * w_br
    return np.clip((acc + 16384) >> 15, 0, 255).astype(np.uint8)


def resize_bilinear_cv2(src, in_h: int, in_w: int, out_h: int, out_w: int) -> np.ndarray:
    """OpenCV's INTER_LINEAR resize for 8-bit images (11-bit coefficients, two passes, 22-bit rounding)."""
    if min(in_h, in_w, out_h, out_w) <= 0:
        raise InferenceError(f"resize_bilinear_cv2: zero dimension - {in_w}x{in_h} -> {out_w}x{out_h}")
    img = _check(src, in_h, in_w, "resize_bilinear_cv2").astype(np.int64)

    def coeffs(n_in, n_out):
        f = (np.arange(n_out, dtype=np.float64) + 0.5) * (n_in / n_out) - 0.5
        s = np.floor(f).astype(np.int64)
        fr = f - s
        lo, hi = s < 0, s >= n_in - 1
        s = np.clip(s, 0, n_in - 1)
        fr = np.where(lo | hi, 0.0, fr)
        return s, np.minimum(s + 1, n_in - 1), np.rint((1.0 - fr) * 2048).astype(np.int64), np.rint(fr * 2048).astype(np.int64)

    x0, x1, wx0, wx1 = coeffs(in_w, out_w)
    y0, y1, wy0, wy1 = coeffs(in_h, out_h)
    hbuf = img[:, x0] * wx0[None, :, None] + img[:, x1] * wx1[None, :, None]            # [in_h, out_w, 3]
    acc = hbuf[y0] * wy0[:, None, None] + hbuf[y1] * wy1[:, None, None]
    return np.clip((acc + (1 << 21)) >> 22, 0, 255).astype(np.uint8)


def norm_crop(src, h: int, w: int, kps) -> np.ndarray:
    return warp_affine(src, h, w, umeyama(np.asarray(kps), ARCFACE_DST), 112, 112)


def align_face_512(src, h: int, w: int, kps) -> np.ndarray:
    return warp_affine(src, h, w, umeyama(np.asarray(kps), FACEXLIB_DST_512), 512, 512, FACEXLIB_BORDER_RGB)


def detector_blob(src, h: int, w: int) -> tuple[torch.Tensor, float]:
    """-> ([1, 3, 640, 640] normalised, scale from image to detector coordinates)."""
    img = _check(src, h, w, "detector_blob")
    ratio = h / w
    new_w, new_h = (int(DET_SIZE / ratio), DET_SIZE) if ratio > 1.0 else (DET_SIZE, int(DET_SIZE * ratio))
    if new_w == 0 or new_h == 0:
        raise InferenceError(f"detector_blob: degenerate aspect ratio {h}x{w}: too far from square for face detection")
    blob = np.full((DET_SIZE, DET_SIZE, 3), (0 - 127.5) / 128.0, dtype=np.float32)
    blob[:new_h, :new_w] = (resize_bilinear_cv2(img, h, w, new_h, new_w).astype(np.float32) - 127.5) / 128.0
    return torch.from_numpy(blob).permute(2, 0, 1)[None].contiguous(), new_h / h


def nms(dets: list[FaceDetection], thresh: float) -> list[FaceDetection]:
    def iou(a, b):
        x1, y1, x2, y2 = max(a[0], b[0]), max(a[1], b[1]), min(a[2], b[2]), min(a[3], b[3])
        inter = max(x2 - x1, 0.0) * max(y2 - y1, 0.0)
        ua = max(a[2] - a[0], 0.0) * max(a[3] - a[1], 0.0) + max(b[2] - b[0], 0.0) * max(b[3] - b[1], 0.0) - inter
        return inter / ua if ua > 0 else 0.0

    keep: list[FaceDetection] = []
    for d in sorted(dets, key=lambda d: -d.score if math.isfinite(d.score) else math.inf):
        if all(iou(k.bbox, d.bbox) <= thresh for k in keep):
            keep.append(d)
    return keep


# ---- networks -----------------------------------------------------------------------------------------------------------
class _ConvNet:
    def __init__(self, weights: dict[str, torch.Tensor], device):
        self.device = torch.device(device)
        self.w = {}
        for k, v in weights.items():
            v = v.float()
            if k.endswith(".weight") and v.dim() == 4:
                v = v.permute(0, 3, 1, 2)                         # stored [out, kh, kw, in]
            self.w[k] = v.to(self.device).contiguous()

    def conv(self, x, name, stride=1, pad=1, relu=False):
        y = F.conv2d(x, self.w[name + ".weight"], self.w[name + ".bias"], stride=stride, padding=pad)
        return F.relu(y) if relu else y


class Scrfd(_ConvNet):
    def _forward(self, x):
        h = self.conv(x, "stem.conv0", 2, 1, True)
        h = self.conv(self.conv(h, "stem.conv1", relu=True), "stem.conv2", relu=True)
        h = F.max_pool2d(h, 2)
        taps = []
        for si, nb in enumerate(SCRFD_STAGES):
            for b in range(nb):
                p = f"stage{si + 1}.{b}"
                down = b == 0 and si > 0
                t = self.conv(self.conv(h, p + ".conv1", 2 if down else 1, 1, True), p + ".conv2")
                ident = self.conv(F.avg_pool2d(h, 2), p + ".downsample", 1, 0) if down else h
                h = F.relu(t + ident)
            taps.append(h)
        c2, c3, c4 = taps[1], taps[2], taps[3]
        l0, l1, l2 = (self.conv(c, f"neck.lateral{i}", 1, 0) for i, c in enumerate((c2, c3, c4)))
        up = lambda t: F.interpolate(t, scale_factor=2.0, mode="nearest")      # noqa: E731
        p4 = l1 + up(l2)
        p3 = l0 + up(p4)
        f0, f1, f2 = self.conv(p3, "neck.fpn0"), self.conv(p4, "neck.fpn1"), self.conv(l2, "neck.fpn2")
        n4 = f1 + self.conv(f0, "neck.down0", 2, 1)
        n5 = f2 + self.conv(n4, "neck.down1", 2, 1)
        feats = {8: f0, 16: self.conv(n4, "neck.pafpn0"), 32: self.conv(n5, "neck.pafpn1")}
        outs = []
        for s, f in feats.items():
            p = f"head{s}"
            h = f
            for j in range(3):
                h = self.conv(h, f"{p}.stem{j}", relu=True)
            flat = lambda t, k: t.permute(0, 2, 3, 1).reshape(-1, k)            # noqa: E731
            outs.append((s, torch.sigmoid(flat(self.conv(h, p + ".cls"), 1)),
                         flat(self.conv(h, p + ".reg"), 4) * float(self.w[p + ".scale"].reshape(-1)[0]),
                         flat(self.conv(h, p + ".kps"), 10)))
        return outs

    @torch.no_grad()
    def detect(self, blob: torch.Tensor, det_scale: float, score_thresh: float = 0.5, nms_thresh: float = 0.4) -> list[FaceDetection]:
        dets = []
        for s, scores, bbox, kps in self._forward(blob.to(self.device)):
            wcells = DET_SIZE // s
            sc = scores[:, 0].cpu().numpy()
            bb, kp = bbox.cpu().numpy(), kps.cpu().numpy()
            for r in np.nonzero(np.isfinite(sc) & (sc >= score_thresh))[0]:
                cell = r // NUM_ANCHORS
                cx, cy = (cell % wcells) * s, (cell // wcells) * s
                d = bb[r]
                box = (cx - d[0] * s, cy - d[1] * s, cx + d[2] * s, cy + d[3] * s)
                pts = [(float(cx + kp[r, 2 * i] * s), float(cy + kp[r, 2 * i + 1] * s)) for i in range(5)]
                dets.append(FaceDetection(tuple(float(v) for v in box), pts, float(sc[r])))
        kept = nms(dets, nms_thresh)
        if det_scale != 1.0:
            inv = 1.0 / det_scale
            kept = [FaceDetection(tuple(v * inv for v in d.bbox), [(x * inv, y * inv) for x, y in d.landmarks], d.score) for d in kept]
        return kept


class ArcFace(_ConvNet):
    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[n, 3, 112, 112] in [-1, 1] -> [n, 512] (raw, not normalised)."""
        w = self.w
        aff = lambda t, p: t * w[p + ".scale"].view(1, -1, 1, 1) + w[p + ".shift"].view(1, -1, 1, 1)     # noqa: E731
        h = F.prelu(self.conv(x.to(self.device), "stem.conv"), w["stem.prelu.weight"].reshape(-1))
        for li, nb in enumerate(ARCFACE_LAYERS):
            for b in range(nb):
                p = f"layer{li + 1}.{b}"
                stride = 2 if b == 0 else 1
                t = F.prelu(self.conv(aff(h, p + ".bn1"), p + ".conv1"), w[p + ".prelu.weight"].reshape(-1))
                t = self.conv(t, p + ".conv2", stride, 1)
                h = t + (self.conv(h, p + ".downsample", stride, 0) if b == 0 else h)
        h = aff(h, "bn2").reshape(h.shape[0], -1)
        h = h @ w["fc.weight"].t() + w["fc.bias"]
        return h * w["features.scale"] + w["features.shift"]


class FaceAnalysis(FaceEmbedder):
    ID = "insightface_antelopev2"

    def __init__(self, scrfd: Scrfd, arcface: ArcFace, backend: str = "cpu"):
        self.scrfd, self.arcface, self.backend = scrfd, arcface, backend
        self.det_thresh, self.nms_thresh = 0.5, 0.4

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor(self.ID, "face", self.backend, {"dim": 512, "landmarks": 5})

    def detect(self, image: Image) -> list[FaceDetection]:
        blob, scale = detector_blob(image.pixels, image.height, image.width)
        dets = self.scrfd.detect(blob, scale, self.det_thresh, self.nms_thresh)
        area = lambda d: max(d.bbox[2] - d.bbox[0], 0.0) * max(d.bbox[3] - d.bbox[1], 0.0)      # noqa: E731
        return sorted(dets, key=lambda d: -area(d))

    def analyze(self, image: Image) -> list[FaceDetection]:
        dets = self.detect(image)
        if not dets:
            return []
        crops = np.stack([norm_crop(image.pixels, image.height, image.width, d.landmarks) for d in dets])
        x = torch.from_numpy((crops.astype(np.float32) - 127.5) / 127.5).permute(0, 3, 1, 2).contiguous()
        emb = self.arcface.forward(x).cpu()
        return [FaceDetection(d.bbox, d.landmarks, d.score, emb[i].tolist()) for i, d in enumerate(dets)]

    def largest_face(self, image: Image) -> FaceDetection:
        faces = self.analyze(image)
        if not faces:
            raise InferenceError(f"{self.ID}: no face detected")
        return faces[0]


def load(root, backend: str = "cpu") -> FaceAnalysis:
    """`root` holds `scrfd.safetensors` and `arcface.safetensors`."""
    from ..io.safetensors_io import load_file

    root = Path(root)
    for f in ("scrfd.safetensors", "arcface.safetensors"):
        if not (root / f).is_file():
            raise LoadError(f"face: {root / f} not found")
    dev = "cuda" if backend == "b200" else "cpu"
    return FaceAnalysis(Scrfd(load_file(root / "scrfd.safetensors"), dev), ArcFace(load_file(root / "arcface.safetensors"), dev), backend)


def random_face_weights(seed: int = 0, width: int = 8) -> tuple[dict[str, torch.Tensor], dict[str, torch.Tensor]]:
    """Random SCRFD / ArcFace weights of the real topology at a small channel width (tests, benchmarks)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)      # noqa: E731

    def conv(w, name, o, i, k):
        w[name + ".weight"], w[name + ".bias"] = rn(o, k, k, i) / math.sqrt(i * k * k), rn(o) * 0.05

    s: dict[str, torch.Tensor] = {}
    c = width
    conv(s, "stem.conv0", c, 3, 3); conv(s, "stem.conv1", c, c, 3); conv(s, "stem.conv2", 2 * c, c, 3)      # noqa: E702
    cin, widths = 2 * c, (2 * c, 4 * c, 6 * c, 8 * c)
    for si, nb in enumerate(SCRFD_STAGES):
        for b in range(nb):
            p = f"stage{si + 1}.{b}"
            conv(s, p + ".conv1", widths[si], cin if b == 0 else widths[si], 3)
            conv(s, p + ".conv2", widths[si], widths[si], 3)
            if b == 0 and si > 0:
                conv(s, p + ".downsample", widths[si], cin, 1)
        cin = widths[si]
    n = 2 * c
    for i, ci in enumerate(widths[1:]):
        conv(s, f"neck.lateral{i}", n, ci, 1)
        conv(s, f"neck.fpn{i}", n, n, 3)
    for i in range(2):
        conv(s, f"neck.down{i}", n, n, 3)
        conv(s, f"neck.pafpn{i}", n, n, 3)
    for st in (8, 16, 32):
        p = f"head{st}"
        for j in range(3):
            conv(s, f"{p}.stem{j}", n, n, 3)
        conv(s, p + ".cls", NUM_ANCHORS, n, 3); conv(s, p + ".reg", 4 * NUM_ANCHORS, n, 3); conv(s, p + ".kps", 10 * NUM_ANCHORS, n, 3)      # noqa: E702
        s[p + ".scale"] = torch.tensor([1.0])
    a: dict[str, torch.Tensor] = {}
    aw = (c, 2 * c, 4 * c, 8 * c)
    conv(a, "stem.conv", c, 3, 3)
    a["stem.prelu.weight"] = torch.full((c,), 0.25)
    cin = c
    for li, nb in enumerate(ARCFACE_LAYERS):
        for b in range(nb):
            p = f"layer{li + 1}.{b}"
            ci = cin if b == 0 else aw[li]
            a[p + ".bn1.scale"], a[p + ".bn1.shift"] = 1.0 + rn(ci) * 0.05, rn(ci) * 0.05
            conv(a, p + ".conv1", aw[li], ci, 3)
            a[p + ".prelu.weight"] = torch.full((aw[li],), 0.25)
            conv(a, p + ".conv2", aw[li], aw[li], 3)
            if b == 0:
                conv(a, p + ".downsample", aw[li], ci, 1)
        cin = aw[li]
    a["bn2.scale"], a["bn2.shift"] = 1.0 + rn(cin) * 0.05, rn(cin) * 0.05
    a["fc.weight"], a["fc.bias"] = rn(512, cin * 7 * 7) / math.sqrt(cin * 49), rn(512) * 0.05
    a["features.scale"], a["features.shift"] = 1.0 + rn(512) * 0.05, rn(512) * 0.05
    return s, a


# ---- face parsing (BiSeNet) ---------------------------------------------------------------------------------------------
BG_LABELS = (0, 16, 18, 7, 8, 9, 14, 15)           # background, cloth, hat, ears, ear-ring, neck-lace, neck: whitened
PARSE_MEAN, PARSE_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
BISENET_FILE = "bisenet_parsing.safetensors"


def upsample_bilinear_align_corners(x: torch.Tensor, out_h: int, out_w: int) -> torch.Tensor:
    """[B, C, h, w] -> [B, C, out_h, out_w] with corner-aligned bilinear weights, as two interpolation matrices."""
    def mat(n_in, n_out):
        m = torch.zeros(n_out, n_in, device=x.device)
        denom = float(max(n_out, 2) - 1)
        for i in range(n_out):
            src = i * (n_in - 1) / denom
            x0 = int(math.floor(src))
            x1 = min(x0 + 1, n_in - 1)
            f = src - x0
            m[i, x0] += 1.0 - f
            m[i, x1] += f
        return m

    return mat(x.shape[2], out_h) @ x @ mat(x.shape[3], out_w).t()


class BiSeNet(_ConvNet):
    """19-class face parsing (parity: candle-gen-face/src/bisenet.rs): ResNet-18 trunk, two attention-refinement
    modules and a global-context vector on the 1/16 and 1/32 features, feature fusion with a squeeze-excite gate at 1/8,
    a 3x3 + 1x1 head, corner-aligned bilinear upsampling to the input size. Batch norms are folded into the
    convolutions of the checkpoint."""

    def _block(self, x, p, stride, down):
        r = self.conv(self.conv(x, p + ".conv1", stride, 1, relu=True), p + ".conv2", 1, 1)
        return F.relu(r + (self.conv(x, p + ".downsample", stride, 0) if down else x))

    def _arm(self, x, p):
        feat = self.conv(x, p + ".conv", 1, 1, relu=True)
        return feat * torch.sigmoid(self.conv(feat.mean((2, 3), keepdim=True), p + ".conv_atten", 1, 0))

    def _conv_w(self, x, name):
        return F.conv2d(x, self.w[name + ".weight"])

    @torch.no_grad()
    def parse_logits(self, x: torch.Tensor) -> torch.Tensor:
        """[B, 3, H, W] ImageNet-normalised -> [B, 19, H, W]."""
        H, W = x.shape[2:]
        h = F.max_pool2d(self.conv(x.to(self.device), "resnet.conv1", 2, 3, relu=True), 3, 2, 1)
        feats = []
        for layer, stride in ((1, 1), (2, 2), (3, 2), (4, 2)):
            h = self._block(h, f"resnet.layer{layer}.0", stride, layer > 1)
            h = self._block(h, f"resnet.layer{layer}.1", 1, False)
            feats.append(h)
        _, f8, f16, f32 = feats
        avg = self.conv(f32.mean((2, 3), keepdim=True), "conv_avg", 1, 0, relu=True)
        s32 = self._arm(f32, "arm32") + avg
        cp16 = self.conv(F.interpolate(s32, size=f16.shape[2:], mode="nearest"), "conv_head32", 1, 1, relu=True)
        s16 = self._arm(f16, "arm16") + cp16
        cp8 = self.conv(F.interpolate(s16, size=f8.shape[2:], mode="nearest"), "conv_head16", 1, 1, relu=True)
        feat = self.conv(torch.cat([f8, cp8], 1), "ffm.convblk", 1, 0, relu=True)
        att = torch.sigmoid(self._conv_w(F.relu(self._conv_w(feat.mean((2, 3), keepdim=True), "ffm.conv1")), "ffm.conv2"))
        fuse = feat * att + feat
        out = self._conv_w(self.conv(fuse, "conv_out.conv", 1, 1, relu=True), "conv_out.conv_out")
        return upsample_bilinear_align_corners(out, H, W)

    def parse_mask(self, x: torch.Tensor) -> torch.Tensor:
        return self.parse_logits(x).argmax(1)


def face_features_image(rgb01: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """[B, 3, H, W] in [0, 1] and a label mask [B, H, W] -> the identity encoder's input: background labels white, the
    rest the luma 0.299 R + 0.587 G + 0.114 B on all three channels."""
    gray = 0.299 * rgb01[:, 0] + 0.587 * rgb01[:, 1] + 0.114 * rgb01[:, 2]
    bg = torch.zeros_like(mask, dtype=torch.bool)
    for lab in BG_LABELS:
        bg |= mask == lab
    v = torch.where(bg.to(gray.device), torch.ones_like(gray), gray)
    return v[:, None].expand(-1, 3, -1, -1).contiguous()


def face_features_for(analysis: FaceAnalysis, parser: BiSeNet, image: Image, face: FaceDetection) -> torch.Tensor:
    """The 512 x 512 aligned crop of `face`, parsed and background-whitened: [1, 3, 512, 512] in [0, 1]."""
    crop = align_face_512(image.pixels, image.height, image.width, face.landmarks)
    rgb01 = torch.from_numpy(crop.astype(np.float32) / 255.0).permute(2, 0, 1)[None].contiguous()
    mean, std = torch.tensor(PARSE_MEAN).view(1, 3, 1, 1), torch.tensor(PARSE_STD).view(1, 3, 1, 1)
    mask = parser.parse_mask((rgb01 - mean) / std).cpu()
    return face_features_image(rgb01, mask)


def random_bisenet_weights(seed: int = 0, width: int = 8) -> dict[str, torch.Tensor]:
    """Random parser weights in the checkpoint's [out, kh, kw, in] layout; `width` scales every channel count
    (64 in the published network)."""
    g = torch.Generator().manual_seed(seed)
    w: dict[str, torch.Tensor] = {}

    def conv(name, o, i, k, bias=True):
        w[name + ".weight"] = torch.randn(o, k, k, i, generator=g) * (1.0 / math.sqrt(i * k * k))
        if bias:
            w[name + ".bias"] = torch.randn(o, generator=g) * 0.01

    c = [width, width, 2 * width, 4 * width, 8 * width]
    conv("resnet.conv1", c[0], 3, 7)
    for layer in range(1, 5):
        cin, cout = c[layer - 1] if layer > 1 else c[0], c[layer]
        conv(f"resnet.layer{layer}.0.conv1", cout, cin, 3)
        conv(f"resnet.layer{layer}.0.conv2", cout, cout, 3)
        if layer > 1:
            conv(f"resnet.layer{layer}.0.downsample", cout, cin, 1)
        conv(f"resnet.layer{layer}.1.conv1", cout, cout, 3)
        conv(f"resnet.layer{layer}.1.conv2", cout, cout, 3)
    m = 2 * width
    for name, cin in (("arm16", c[3]), ("arm32", c[4])):
        conv(name + ".conv", m, cin, 3)
        conv(name + ".conv_atten", m, m, 1)
    conv("conv_head32", m, m, 3)
    conv("conv_head16", m, m, 3)
    conv("conv_avg", m, c[4], 1)
    conv("ffm.convblk", 2 * m, c[2] + m, 1)
    conv("ffm.conv1", m // 2, 2 * m, 1, bias=False)
    conv("ffm.conv2", 2 * m, m // 2, 1, bias=False)
    conv("conv_out.conv", 2 * m, 2 * m, 3)
    conv("conv_out.conv_out", 19, 2 * m, 1, bias=False)
    return w
