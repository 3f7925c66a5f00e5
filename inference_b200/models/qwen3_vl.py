"""Qwen3-VL: vision tower with DeepStack taps, three-axis position ids and interleaved M-RoPE tables
(parity: candle-llm/src/models/qwen35_vision.rs, deepstack.rs; checkpoint keys are the Hugging Face `model.visual.*`
names).

Vision tower: patches of 2 frames x 16 x 16 pixels (a still image repeats its frame) go through a linear patch
embedding; a learned 48 x 48 position table is bilinearly resampled to the image's patch grid; blocks are pre-LayerNorm
attention (2-D rotary positions, full attention inside one frame) + GELU-tanh MLP. Tokens are ordered so that every
2 x 2 spatial group is contiguous, and the merger turns each group into one language-model token. Three intermediate
layers are tapped through their own mergers (DeepStack); the decoder adds tap i to the image positions of its
residual stream after decoder layer i.

Decoder side: an image occupies positions (start, start + row, start + col) on the (t, h, w) axes and the next text
token continues at start + max(rows, cols); the rotary table takes frequency j from axis j % 3 while j < 3 * section
(h, w) and from t otherwise."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class Qwen3VlVisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: tuple[int, ...] = (8, 16, 24)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def grid_side(self) -> int:
        return int(round(math.sqrt(self.num_position_embeddings)))

    @staticmethod
    def from_json(j: dict) -> "Qwen3VlVisionConfig":
        j = j.get("vision_config", j)
        d = {k: j[k] for k in Qwen3VlVisionConfig.__dataclass_fields__ if k in j}
        if "deepstack_visual_indexes" in d:
            d["deepstack_visual_indexes"] = tuple(d["deepstack_visual_indexes"])
        return Qwen3VlVisionConfig(**d)


def merge_order(h: int, w: int, m: int) -> torch.Tensor:
    """Row-major patch indices of an h x w grid, listed so that every m x m group is contiguous."""
    return torch.arange(h * w).view(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)


class Qwen3VlVisionTower:
    def __init__(self, cfg: Qwen3VlVisionConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32,
                 prefix: str = "model.visual."):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k[len(prefix):]: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()
                  if k.startswith(prefix)}
        self.w["patch_embed.proj.weight"] = self.w["patch_embed.proj.weight"].reshape(cfg.hidden_size, -1).contiguous()

    def _lin(self, x, name):
        from .text_encoders import linear

        return linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            1e-6).to(x.dtype)

    def position_table(self, h: int, w: int) -> torch.Tensor:
        """The learned grid resampled bilinearly (corner-aligned) to h x w patches, row-major [h*w, hidden]."""
        side = self.cfg.grid_side
        table = self.w["pos_embed.weight"].float().view(side, side, -1)
        ys, xs = torch.linspace(0, side - 1, h, device=self.device), torch.linspace(0, side - 1, w, device=self.device)
        y0, x0 = ys.floor().long(), xs.floor().long()
        y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
        fy, fx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
        out = (table[y0][:, x0] * (1 - fy) * (1 - fx) + table[y0][:, x1] * (1 - fy) * fx
               + table[y1][:, x0] * fy * (1 - fx) + table[y1][:, x1] * fy * fx)
        return out.reshape(h * w, -1).to(self.dtype)

    def rotary_table(self, h: int, w: int) -> tuple[torch.Tensor, torch.Tensor]:
        """cos / sin [h*w, head_dim] in row-major patch order: the first quarter of the frequencies turns with the
        row, the second with the column, and the pair is repeated for the rotate-half layout."""
        q = self.cfg.head_dim // 4
        inv = 1.0 / (10000.0 ** (torch.arange(q, dtype=torch.float32, device=self.device) * 2 / (2 * q)))
        rows = torch.arange(h, device=self.device, dtype=torch.float32).repeat_interleave(w)
        cols = torch.arange(w, device=self.device, dtype=torch.float32).repeat(h)
        ang = torch.cat([rows[:, None] * inv, cols[:, None] * inv], -1)
        ang = torch.cat([ang, ang], -1)
        return ang.cos(), ang.sin()

    def _merger(self, x, p, post_shuffle: bool):
        g = self.cfg.spatial_merge_size ** 2
        if post_shuffle:
            x = self._ln(x.reshape(-1, g * x.shape[-1]), p + ".norm")
        else:
            x = self._ln(x, p + ".norm").reshape(-1, g * x.shape[-1])
        return self._lin(F.gelu(self._lin(x, p + ".linear_fc1").float()).to(x.dtype), p + ".linear_fc2")

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grid_thw: list[tuple[int, int, int]]
                ) -> tuple[torch.Tensor, list[torch.Tensor]]:
        """patches [N, patch_dim] in merge order (every image: frames, then 2 x 2 groups), grid_thw one (t, h, w) per
        image in patches -> (tokens [N / 4, out_hidden], one [N / 4, out_hidden] tensor per DeepStack tap)."""
        cfg = self.cfg
        m, nh, hd = cfg.spatial_merge_size, cfg.num_heads, cfg.head_dim
        x = self._lin(patches.to(self.device, self.dtype), "patch_embed.proj")
        pos, cos, sin, spans = [], [], [], []
        start = 0
        for t, h, w in grid_thw:
            order = merge_order(h, w, m).to(self.device)
            c, s = self.rotary_table(h, w)
            pos.append(self.position_table(h, w)[order].repeat(t, 1))
            cos.append(c[order].repeat(t, 1))
            sin.append(s[order].repeat(t, 1))
            for _ in range(t):                       # attention is full inside one frame and blind across frames
                spans.append((start, start + h * w))
                start += h * w
        x = x + torch.cat(pos, 0)
        cos, sin = torch.cat(cos, 0)[:, None, :], torch.cat(sin, 0)[:, None, :]
        taps = []
        for i in range(cfg.depth):
            p = f"blocks.{i}"
            q, k, v = self._lin(self._ln(x, p + ".norm1"), p + ".attn.qkv").view(-1, 3, nh, hd).float().unbind(1)

            def rot(u):
                u1, u2 = u[..., : hd // 2], u[..., hd // 2:]
                return u * cos + torch.cat([-u2, u1], -1) * sin
            q, k = rot(q), rot(k)
            out = torch.empty_like(q)
            for a, b in spans:
                out[a:b] = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                                          v[a:b].transpose(0, 1)[None])[0].transpose(0, 1)
            x = x + self._lin(out.reshape(-1, nh * hd).to(self.dtype), p + ".attn.proj")
            h2 = F.gelu(self._lin(self._ln(x, p + ".norm2"), p + ".mlp.linear_fc1").float(), approximate="tanh")
            x = x + self._lin(h2.to(self.dtype), p + ".mlp.linear_fc2")
            if i in cfg.deepstack_visual_indexes:
                taps.append(self._merger(x, f"deepstack_merger_list.{cfg.deepstack_visual_indexes.index(i)}", True))
        return self._merger(x, "merger", False), taps


# ---- image -> patches --------------------------------------------------------------------------------------------------------
def smart_resize(height: int, width: int, factor: int = 32, min_pixels: int = 256 * 256, max_pixels: int = 1280 * 1280
                 ) -> tuple[int, int]:
    """The size closest to (height, width) with both sides multiples of `factor` and an area inside the limits."""
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def image_to_patches(rgb: torch.Tensor, cfg: Qwen3VlVisionConfig, **limits) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """uint8 [H, W, 3] -> (patches [h*w, patch_dim] in merge order, (1, h, w)): bicubic resize to the smart size,
    (x / 255 - 0.5) / 0.5, the frame repeated to fill the temporal patch."""
    P, m, T = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    H, W = smart_resize(rgb.shape[0], rgb.shape[1], P * m, **limits)
    x = rgb.permute(2, 0, 1)[None].float()
    if (H, W) != tuple(rgb.shape[:2]):
        x = F.interpolate(x, size=(H, W), mode="bicubic", align_corners=False, antialias=True).clamp(0, 255)
    x = (x[0] / 255.0 - 0.5) / 0.5                                      # [3, H, W]
    h, w = H // P, W // P
    x = x.view(3, h // m, m, P, w // m, m, P).permute(1, 4, 2, 5, 0, 3, 6)          # [h/m, w/m, m, m, 3, P, P]
    x = x[:, :, :, :, :, None].expand(-1, -1, -1, -1, -1, T, -1, -1)
    return x.reshape(h * w, cfg.patch_dim).contiguous(), (1, h, w)


def video_to_patches(frames: list[torch.Tensor], timestamps: list[float], cfg: Qwen3VlVisionConfig, **limits
                     ) -> tuple[torch.Tensor, tuple[int, int, int], list[float]]:
    """uint8 [H, W, 3] frames -> (patches [t*h*w, patch_dim] in merge order, (t, h, w), one timestamp per temporal patch).
    Frames are grouped in pairs (the last frame repeats when the count is odd); a pair's timestamp is the mean of its
    frames' times."""
    P, m, T = cfg.patch_size, cfg.spatial_merge_size, cfg.temporal_patch_size
    frames, timestamps = list(frames), list(timestamps)
    while len(frames) % T:
        frames.append(frames[-1])
        timestamps.append(timestamps[-1])
    H, W = smart_resize(frames[0].shape[0], frames[0].shape[1], P * m, **limits)
    h, w = H // P, W // P
    px = []
    for f in frames:
        x = f.permute(2, 0, 1)[None].float()
        if (H, W) != tuple(f.shape[:2]):
            x = F.interpolate(x, size=(H, W), mode="bicubic", align_corners=False, antialias=True).clamp(0, 255)
        px.append((x[0] / 255.0 - 0.5) / 0.5)
    v = torch.stack(px, 0).view(len(frames) // T, T, 3, h // m, m, P, w // m, m, P)
    v = v.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)                                  # [t, h/m, w/m, m, m, 3, T, P, P]
    t = len(frames) // T
    stamps = [sum(timestamps[i * T:(i + 1) * T]) / T for i in range(t)]
    return v.reshape(t * h * w, cfg.patch_dim).contiguous(), (t, h, w), stamps


def video_placeholder_text(stamps: list[float]) -> str:
    """One vision run per temporal patch, each announced by its time: `<0.2 seconds><|vision_start|><|video_pad|><|vision_end|>`."""
    return "".join(f"<{s:.1f} seconds><|vision_start|><|video_pad|><|vision_end|>" for s in stamps)


# ---- decoder side ------------------------------------------------------------------------------------------------------------
def mrope_positions(ids: list[int], grids: list[tuple[int, int, int]], image_token_id, merge: int = 2
                    ) -> tuple[torch.Tensor, int]:
    """(positions [3, S], next position) for a prompt whose runs of vision placeholder tokens are, in order, the grids
    of `grids` (t, h, w before merging). `image_token_id` is one id or a collection (image and video placeholders); a
    video contributes one (1, h, w) grid per temporal patch, since every patch is its own run behind its timestamp."""
    vision = {image_token_id} if isinstance(image_token_id, int) else set(image_token_id)
    pos = torch.zeros(3, len(ids), dtype=torch.int64)
    nxt, i, g = 0, 0, 0
    while i < len(ids):
        if ids[i] not in vision:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        t, h, w = grids[g]
        g += 1
        rows, cols = h // merge, w // merge
        n = t * rows * cols
        if len(set(ids[i:i + n])) != 1 or len(ids[i:i + n]) != n:
            raise ValueError(f"image {g - 1} needs a run of {n} placeholder tokens at position {i}")
        pos[0, i:i + n] = nxt
        pos[1, i:i + n] = nxt + torch.arange(rows).repeat_interleave(cols).repeat(t)
        pos[2, i:i + n] = nxt + torch.arange(cols).repeat(rows * t)
        nxt += max(rows, cols)
        i += n
    return pos, nxt


def interleaved_mrope_table(positions: torch.Tensor, inv_freq: torch.Tensor, section: tuple[int, int, int]
                            ) -> tuple[torch.Tensor, torch.Tensor]:
    """positions [3, S] -> cos / sin [S, len(inv_freq)]: frequency j follows the h axis when j % 3 == 1 and
    j < 3 * section[1], the w axis when j % 3 == 2 and j < 3 * section[2], the t axis otherwise."""
    n = inv_freq.numel()
    j = torch.arange(n, device=inv_freq.device)
    axis = torch.zeros(n, dtype=torch.int64, device=inv_freq.device)
    axis[(j % 3 == 1) & (j < 3 * section[1])] = 1
    axis[(j % 3 == 2) & (j < 3 * section[2])] = 2
    ang = positions.to(inv_freq.device).float()[axis, :].t() * inv_freq.float()[None, :]          # [S, n]
    return ang.cos(), ang.sin()


def language_model_config(j: dict):
    """The language tower of a Qwen3-VL checkpoint as a plain Qwen3 decoder configuration (for callers that use the
    tower as a text / instruction encoder): the `text_config` block, dense or mixture-of-experts, with its rotary
    parameters (the three M-RoPE sections coincide on text-only prompts)."""
    from .config import ModelConfig

    t = dict(j.get("text_config", j))
    moe = bool(t.get("num_experts"))
    t["architectures"] = ["Qwen3MoeForCausalLM" if moe else "Qwen3ForCausalLM"]
    t["model_type"] = "qwen3_moe" if moe else "qwen3"
    t.setdefault("tie_word_embeddings", j.get("tie_word_embeddings", False))
    return ModelConfig.from_json(t)
