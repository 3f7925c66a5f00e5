"""Depth Anything V2: DINOv2 backbone + DPT neck / head, the reference's depth utility
(candle-gen-depth: Depth-Anything V2). Weight names follow the Hugging Face `DepthAnythingForDepthEstimation`
checkpoint (`backbone.embeddings...`, `backbone.encoder.layer.N...`, `neck.reassemble_stage.layers.N...`,
`neck.fusion_stage.layers.N...`, `head.conv1...`).

The transformer's projections run on the tcgen05 GEMM for bf16 weights on a CUDA device; the neck's small convolutions
and bilinear resizes are torch ops."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .text_encoders import linear


@dataclass
class DepthConfig:
    hidden_size: int = 384
    num_hidden_layers: int = 12
    num_attention_heads: int = 6
    mlp_ratio: int = 4
    patch_size: int = 14
    image_size: int = 518
    layer_norm_eps: float = 1e-6
    out_indices: list[int] = field(default_factory=lambda: [3, 6, 9, 12])
    apply_layernorm: bool = True
    reassemble_hidden_size: int = 384
    reassemble_factors: list[float] = field(default_factory=lambda: [4, 2, 1, 0.5])
    neck_hidden_sizes: list[int] = field(default_factory=lambda: [48, 96, 192, 384])
    fusion_hidden_size: int = 64
    head_in_index: int = -1
    head_hidden_size: int = 32
    depth_estimation_type: str = "relative"
    max_depth: float = 1.0

    @staticmethod
    def from_json(j: dict) -> "DepthConfig":
        b = j.get("backbone_config") or {}
        c = DepthConfig()
        for k in ("hidden_size", "num_hidden_layers", "num_attention_heads", "mlp_ratio", "patch_size", "image_size",
                  "layer_norm_eps", "apply_layernorm"):
            if k in b:
                setattr(c, k, b[k])
        if b.get("out_indices"):
            c.out_indices = list(b["out_indices"])
        elif b.get("out_features"):
            c.out_indices = [int(s.replace("stage", "")) for s in b["out_features"]]
        for k in ("reassemble_hidden_size", "reassemble_factors", "neck_hidden_sizes", "fusion_hidden_size",
                  "head_in_index", "head_hidden_size", "depth_estimation_type"):
            if k in j:
                setattr(c, k, j[k])
        if j.get("max_depth") is not None:
            c.max_depth = float(j["max_depth"])
        c.patch_size = int(j.get("patch_size", c.patch_size))
        return c


class DepthAnything:
    def __init__(self, cfg: DepthConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype).contiguous() for k, v in weights.items() if v.is_floating_point()}
        pw = self.w["backbone.embeddings.patch_embeddings.projection.weight"]
        self._patch_w = pw.reshape(pw.shape[0], -1).contiguous()

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            self.cfg.layer_norm_eps).to(self.dtype)

    def _conv(self, x, name, **kw):
        return F.conv2d(x, self.w[name + ".weight"], self.w.get(name + ".bias"), **kw)

    def _pos(self, n_h: int, n_w: int) -> torch.Tensor:
        pe = self.w["backbone.embeddings.position_embeddings"]
        n = pe.shape[1] - 1
        if n == n_h * n_w and n_h == n_w:
            return pe
        s = int(n ** 0.5)
        grid = pe[:, 1:].reshape(1, s, s, -1).permute(0, 3, 1, 2).float()
        grid = F.interpolate(grid, size=(n_h, n_w), mode="bicubic", align_corners=False).to(pe.dtype)
        return torch.cat([pe[:, :1], grid.permute(0, 2, 3, 1).reshape(1, n_h * n_w, -1)], dim=1)

    @torch.no_grad()
    def backbone(self, pixels: torch.Tensor) -> list[torch.Tensor]:
        """[B, 3, H, W] (multiples of the patch size) -> the token states (class token first) after the configured
        layers, layer-normed."""
        c = self.cfg
        B, _, Hh, Ww = pixels.shape
        P = c.patch_size
        nh, nw = Hh // P, Ww // P
        cols = F.unfold(pixels.to(self.device, self.dtype), kernel_size=P, stride=P).transpose(1, 2)
        x = linear(cols, self._patch_w, self.w["backbone.embeddings.patch_embeddings.projection.bias"])
        x = torch.cat([self.w["backbone.embeddings.cls_token"].expand(B, 1, -1), x], dim=1) + self._pos(nh, nw)
        H = c.num_attention_heads
        outs = []
        for i in range(c.num_hidden_layers):
            p = f"backbone.encoder.layer.{i}."
            h = self._ln(x, p + "norm1")
            q, k, v = (linear(h, self.w[f"{p}attention.attention.{n}.weight"], self.w[f"{p}attention.attention.{n}.bias"])
                       for n in ("query", "key", "value"))
            sp = lambda t: t.view(B, -1, H, t.shape[-1] // H).transpose(1, 2)
            a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(1, 2).reshape(x.shape)
            a = linear(a, self.w[p + "attention.output.dense.weight"], self.w[p + "attention.output.dense.bias"])
            x = x + a * self.w[p + "layer_scale1.lambda1"]
            h = self._ln(x, p + "norm2")
            h = F.gelu(linear(h, self.w[p + "mlp.fc1.weight"], self.w[p + "mlp.fc1.bias"]).float()).to(self.dtype)
            x = x + linear(h, self.w[p + "mlp.fc2.weight"], self.w[p + "mlp.fc2.bias"]) * self.w[p + "layer_scale2.lambda1"]
            if i + 1 in c.out_indices:
                outs.append(self._ln(x, "backbone.layernorm") if c.apply_layernorm else x)
        return outs

    def _residual_unit(self, x, p):
        h = self._conv(F.relu(x), p + ".convolution1", padding=1)
        return self._conv(F.relu(h), p + ".convolution2", padding=1) + x

    @torch.no_grad()
    def predict(self, pixels: torch.Tensor) -> torch.Tensor:
        """Depth map [B, H, W] (relative models: larger = closer, unbounded; metric ones: metres up to max_depth)."""
        c = self.cfg
        B, _, Hh, Ww = pixels.shape
        nh, nw = Hh // c.patch_size, Ww // c.patch_size
        feats = []
        for i, hs in enumerate(self.backbone(pixels)):
            f = hs[:, 1:].reshape(B, nh, nw, -1).permute(0, 3, 1, 2).contiguous()
            p = f"neck.reassemble_stage.layers.{i}"
            f = self._conv(f, p + ".projection")
            factor = c.reassemble_factors[i]
            if factor > 1:
                f = F.conv_transpose2d(f, self.w[p + ".resize.weight"], self.w.get(p + ".resize.bias"), stride=int(factor))
            elif factor < 1:
                f = self._conv(f, p + ".resize", stride=int(1 / factor), padding=1)
            feats.append(self._conv(f, f"neck.convs.{i}", padding=1))
        feats = feats[::-1]
        fused, outs = None, []
        for idx, f in enumerate(feats):
            p = f"neck.fusion_stage.layers.{idx}"
            size = feats[idx + 1].shape[2:] if idx != len(feats) - 1 else None
            if fused is None:
                h = f
            else:
                r = f if f.shape == fused.shape else F.interpolate(f, size=fused.shape[2:], mode="bilinear",
                                                                   align_corners=False)
                h = fused + self._residual_unit(r, p + ".residual_layer1")
            h = self._residual_unit(h, p + ".residual_layer2")
            h = F.interpolate(h, size=tuple(size), mode="bilinear", align_corners=True) if size is not None else \
                F.interpolate(h, scale_factor=2, mode="bilinear", align_corners=True)
            fused = self._conv(h, p + ".projection")
            outs.append(fused)
        d = self._conv(outs[c.head_in_index], "head.conv1", padding=1)
        d = F.interpolate(d, (nh * c.patch_size, nw * c.patch_size), mode="bilinear", align_corners=True)
        d = F.relu(self._conv(d, "head.conv2", padding=1))
        d = self._conv(d, "head.conv3")
        d = (F.relu(d) if c.depth_estimation_type == "relative" else torch.sigmoid(d)) * c.max_depth
        return d.squeeze(1)


IMAGENET_MEAN, IMAGENET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


def preprocess(rgb8: torch.Tensor, target: int = 518, patch: int = 14) -> torch.Tensor:
    """uint8 [H, W, 3] -> [1, 3, h, w]: the short side is scaled to `target` keeping the aspect ratio, both sides are
    rounded to multiples of the patch size (bicubic), then ImageNet normalisation."""
    x = rgb8.permute(2, 0, 1).unsqueeze(0).float() / 255.0
    h, w = x.shape[2:]
    s = target / min(h, w)
    nh, nw = max(patch, round(h * s / patch) * patch), max(patch, round(w * s / patch) * patch)
    x = F.interpolate(x, size=(nh, nw), mode="bicubic", align_corners=False).clamp(0, 1)
    m, sd = torch.tensor(IMAGENET_MEAN).view(1, 3, 1, 1), torch.tensor(IMAGENET_STD).view(1, 3, 1, 1)
    return (x - m) / sd
