"""Vision transformer towers: CLIP ViT (class token, pre-LayerNorm, quick-GELU) and SigLIP (no class token,
tanh-GELU, attention-pooling head), the image side of the reference's embedders and its LLaVA captioner
(candle-gen-clip `clip_vit_l14`; candle-gen-joycaption's SigLIP + Llama-3.1-8B).

Weight names follow the Hugging Face checkpoints (`vision_model.embeddings.patch_embedding.weight`,
`vision_model.encoder.layers.N.self_attn.q_proj.weight`, ...). Projections go through the tcgen05 GEMM for bf16
weights on a CUDA device (`text_encoders.linear`); the patch embedding is a strided convolution evaluated as
unfold + GEMM, so it takes the same path."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .text_encoders import linear


@dataclass
class VisionConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 224
    patch_size: int = 14
    num_channels: int = 3
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"
    projection_dim: int | None = None
    kind: str = "clip"                  # "clip" | "siglip"

    @staticmethod
    def from_json(j: dict, kind: str | None = None) -> "VisionConfig":
        src = j.get("vision_config", j)
        keys = VisionConfig.__dataclass_fields__
        cfg = VisionConfig(**{k: src[k] for k in keys if k in src and k != "kind"})
        if "vision_config" in j and "projection_dim" in j:      # the joint model's width wins over the tower's default
            cfg.projection_dim = j["projection_dim"]
        mt = (kind or src.get("model_type") or j.get("model_type") or "clip").lower()
        cfg.kind = "siglip" if "siglip" in mt else "clip"
        return cfg

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2


def _act(x: torch.Tensor, name: str) -> torch.Tensor:
    x = x.float()
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    return F.gelu(x)


class VisionTower:
    def __init__(self, cfg: VisionConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()
                  if k.startswith(("vision_model.", "visual_projection."))}
        pw = self.w["vision_model.embeddings.patch_embedding.weight"]
        self._patch_w = pw.reshape(pw.shape[0], -1).contiguous()       # [hidden, C * P * P]

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            self.cfg.layer_norm_eps).to(self.dtype)

    def _mha(self, q, k, v, H):
        B, Lq, E = q.shape
        D = E // H
        sp = lambda t: t.view(B, -1, H, D).transpose(1, 2)
        o = F.scaled_dot_product_attention(sp(q), sp(k), sp(v))
        return o.transpose(1, 2).reshape(B, Lq, E)

    @torch.no_grad()
    def hidden_states(self, pixels: torch.Tensor, layer: int = -1) -> torch.Tensor:
        """pixels [B, 3, S, S] (already normalised) -> token states [B, tokens, hidden] after encoder layer `layer`
        (negative counts from the end; -1 is the last layer, -2 the penultimate one LLaVA-style models read),
        before any final LayerNorm."""
        cfg = self.cfg
        p = "vision_model."
        B = pixels.shape[0]
        P = cfg.patch_size
        cols = F.unfold(pixels.to(self.device, self.dtype), kernel_size=P, stride=P).transpose(1, 2)   # [B, N, C*P*P]
        x = linear(cols, self._patch_w, self.w.get(p + "embeddings.patch_embedding.bias"))
        if cfg.kind == "clip":
            cls = self.w[p + "embeddings.class_embedding"].expand(B, 1, -1)
            x = torch.cat([cls, x], dim=1)
        x = x + self.w[p + "embeddings.position_embedding.weight"][: x.shape[1]]
        if cfg.kind == "clip":
            x = self._ln(x, p + ("pre_layrnorm" if p + "pre_layrnorm.weight" in self.w else "pre_layernorm"))
        n = cfg.num_hidden_layers
        upto = n + 1 + layer if layer < 0 else layer
        H = cfg.num_attention_heads
        for i in range(upto):
            lp = f"{p}encoder.layers.{i}."
            h = self._ln(x, lp + "layer_norm1")
            q, k, v = (linear(h, self.w[f"{lp}self_attn.{m}_proj.weight"], self.w[f"{lp}self_attn.{m}_proj.bias"])
                       for m in "qkv")
            x = x + linear(self._mha(q, k, v, H), self.w[lp + "self_attn.out_proj.weight"],
                           self.w[lp + "self_attn.out_proj.bias"])
            h = self._ln(x, lp + "layer_norm2")
            h = _act(linear(h, self.w[lp + "mlp.fc1.weight"], self.w[lp + "mlp.fc1.bias"]), cfg.hidden_act).to(self.dtype)
            x = x + linear(h, self.w[lp + "mlp.fc2.weight"], self.w[lp + "mlp.fc2.bias"])
        return x

    @torch.no_grad()
    def pooled(self, pixels: torch.Tensor) -> torch.Tensor:
        """CLIP: post-LayerNorm of the class token. SigLIP: the attention-pooling head (a learned probe attends over
        the normed tokens, then an MLP residual)."""
        cfg = self.cfg
        p = "vision_model."
        x = self.hidden_states(pixels)
        if cfg.kind == "clip":
            return self._ln(x[:, 0], p + "post_layernorm")
        x = self._ln(x, p + "post_layernorm")
        hp = p + "head."
        E = cfg.hidden_size
        wi, bi = self.w[hp + "attention.in_proj_weight"], self.w[hp + "attention.in_proj_bias"]
        probe = self.w[hp + "probe"].expand(x.shape[0], 1, -1)
        q = linear(probe, wi[:E].contiguous(), bi[:E].contiguous())
        k = linear(x, wi[E:2 * E].contiguous(), bi[E:2 * E].contiguous())
        v = linear(x, wi[2 * E:].contiguous(), bi[2 * E:].contiguous())
        a = linear(self._mha(q, k, v, cfg.num_attention_heads), self.w[hp + "attention.out_proj.weight"],
                   self.w[hp + "attention.out_proj.bias"])
        h = self._ln(a, hp + "layernorm")
        h = _act(linear(h, self.w[hp + "mlp.fc1.weight"], self.w[hp + "mlp.fc1.bias"]), cfg.hidden_act).to(self.dtype)
        return (a + linear(h, self.w[hp + "mlp.fc2.weight"], self.w[hp + "mlp.fc2.bias"]))[:, 0]

    @torch.no_grad()
    def image_embeds(self, pixels: torch.Tensor) -> torch.Tensor:
        """The joint-space embedding: pooled state through `visual_projection` when the checkpoint has one."""
        x = self.pooled(pixels)
        w = self.w.get("visual_projection.weight")
        return linear(x, w) if w is not None else x


CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
SIGLIP_MEAN, SIGLIP_STD = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)


def preprocess(rgb8: torch.Tensor, size: int, mean=CLIP_MEAN, std=CLIP_STD, crop: bool = True) -> torch.Tensor:
    """uint8 [H, W, 3] -> float [1, 3, size, size]: bicubic resize of the short side (CLIP) or of both sides
    (crop=False, SigLIP), centre crop, scale to [0, 1], normalise."""
    x = rgb8.permute(2, 0, 1).unsqueeze(0).float()
    h, w = x.shape[2:]
    if crop:
        s = size / min(h, w)
        nh, nw = max(size, round(h * s)), max(size, round(w * s))
        x = F.interpolate(x, size=(nh, nw), mode="bicubic", align_corners=False, antialias=True).clamp(0, 255)
        t, l = (nh - size) // 2, (nw - size) // 2
        x = x[:, :, t:t + size, l:l + size]
    else:
        x = F.interpolate(x, size=(size, size), mode="bicubic", align_corners=False, antialias=True).clamp(0, 255)
    x = x.round() / 255.0
    m, s = torch.tensor(mean).view(1, 3, 1, 1), torch.tensor(std).view(1, 3, 1, 1)
    return (x - m) / s


def random_vision_weights(cfg: VisionConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """A random CLIP-style vision tower (class token, pre / post LayerNorm, optional visual projection)."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)      # noqa: E731
    E, I, P = cfg.hidden_size, cfg.intermediate_size, cfg.patch_size
    p = "vision_model."
    w = {p + "embeddings.patch_embedding.weight": rn(E, cfg.num_channels, P, P) * std,
         p + "embeddings.class_embedding": rn(E) * std,
         p + "embeddings.position_embedding.weight": rn(cfg.num_patches + 1, E) * std}
    for n in ("pre_layrnorm", "post_layernorm"):
        w[p + n + ".weight"], w[p + n + ".bias"] = 1.0 + rn(E) * 0.05, rn(E) * 0.02
    for i in range(cfg.num_hidden_layers):
        lp = f"{p}encoder.layers.{i}."
        for n in ("layer_norm1", "layer_norm2"):
            w[lp + n + ".weight"], w[lp + n + ".bias"] = 1.0 + rn(E) * 0.05, rn(E) * 0.02
        for m in ("q_proj", "k_proj", "v_proj", "out_proj"):
            w[f"{lp}self_attn.{m}.weight"], w[f"{lp}self_attn.{m}.bias"] = rn(E, E) * std, rn(E) * 0.01
        w[lp + "mlp.fc1.weight"], w[lp + "mlp.fc1.bias"] = rn(I, E) * std, rn(I) * 0.01
        w[lp + "mlp.fc2.weight"], w[lp + "mlp.fc2.bias"] = rn(E, I) * std, rn(E) * 0.01
    if cfg.projection_dim:
        w["visual_projection.weight"] = rn(cfg.projection_dim, E) * std
    return w
