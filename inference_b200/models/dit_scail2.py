"""SCAIL-2 animation DiT and its CLIP image tower (parity: candle-gen-scail2/src/{model,rope,clip,common,config}.rs;
checkpoint keys are the original Wan names: `blocks.N.self_attn.q`, `cross_attn.k_img`, `ffn.0`, `modulation`, `head.head`).

A Wan2.1-14B image-to-video network with packed-token conditioning. One token sequence holds, in order: extra
reference characters (optional), the reference image, the noisy target clip, and the driving (pose) clip at half
resolution. Latents are widened to 20 channels by a 4-channel flag (ones for clean inputs and for history frames, zeros
for the frames being denoised); a 28-channel colour-class mask (7 classes x 4 sub-frames) is patch-embedded by its own
stem and ADDED to the latent embedding of the same tokens; the pose clip has its own stem. Each chunk has its own rotary
offsets: reference frames sit before the video in time (and 120 rows down in replacement mode), the pose chunk 120
columns right with every rotary entry the average over the 2 x 2 positions it covers. Cross-attention attends the text
and, through extra k / v projections, 257 CLIP ViT-H/14 tokens of the reference image; the two results are summed.
Only the target clip's tokens are read back.

One implementation for both backends (nn_dual): fp32 oracle on CPU; bf16 with tcgen05 GEMM / attention on a CUDA device."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

ROPE_THETA, IMG_LN_EPS = 10000.0, 1e-5


@dataclass
class Scail2Config:
    dim: int = 5120
    ffn_dim: int = 13824
    num_heads: int = 40
    num_layers: int = 40
    in_dim: int = 20
    out_dim: int = 16
    mask_dim: int = 28
    i2v_mask_dim: int = 4
    freq_dim: int = 256
    text_len: int = 512
    text_dim: int = 4096
    eps: float = 1e-6
    patch: tuple = (1, 2, 2)
    vae_z_dim: int = 16
    replace_h_shift: int = 120
    pose_w_shift: int = 120
    clip_dim: int = 1280

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads

    @staticmethod
    def from_json(j: dict) -> "Scail2Config":
        c = Scail2Config()
        for k in ("in_dim", "out_dim", "dim", "ffn_dim", "num_heads", "num_layers", "mask_dim", "text_dim", "text_len", "freq_dim",
                  "clip_dim", "replace_h_shift", "pose_w_shift"):
            if isinstance(j.get(k), int):
                setattr(c, k, j[k])
        return c


class ScailRope:
    """Three-axis adjacent-pair rotary table with the Wan lane split (head 128: 22 time, 21 row, 21 column pairs)."""

    def __init__(self, head_dim: int):
        d6 = head_dim // 6
        t_dim, a_dim = head_dim - 4 * d6, 2 * d6
        self.inv_t = ROPE_THETA ** (-torch.arange(0, t_dim, 2, dtype=torch.float64) / t_dim)
        self.inv_a = ROPE_THETA ** (-torch.arange(0, a_dim, 2, dtype=torch.float64) / a_dim)
        self.half_d = self.inv_t.numel() + 2 * self.inv_a.numel()

    def chunk(self, grid, shift=(0, 0, 0), pose_downsample: bool = False):
        """cos / sin [f * h * w (or f * h/2 * w/2), half_d] of a (frames, rows, columns) grid offset by `shift`."""
        f, h, w = grid
        pos = torch.stack(torch.meshgrid(torch.arange(f, dtype=torch.float64) + shift[0], torch.arange(h, dtype=torch.float64) + shift[1],
                                         torch.arange(w, dtype=torch.float64) + shift[2], indexing="ij"), -1)      # [f, h, w, 3]
        ang = torch.cat([pos[..., 0:1] * self.inv_t, pos[..., 1:2] * self.inv_a, pos[..., 2:3] * self.inv_a], -1)
        cos, sin = ang.cos().float(), ang.sin().float()
        if pose_downsample:
            pool = lambda t: t.reshape(f, h // 2, 2, w // 2, 2, -1).mean((2, 4))                # noqa: E731
            cos, sin = pool(cos[:, :h // 2 * 2, :w // 2 * 2]), pool(sin[:, :h // 2 * 2, :w // 2 * 2])
        return cos.reshape(-1, self.half_d), sin.reshape(-1, self.half_d)


def patchify(x: torch.Tensor, patch) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """[C, T, H, W] -> ([tokens, C * pt * ph * pw] in the patch convolution's weight order, the token grid)."""
    C, T, H, W = x.shape
    pt, ph, pw = patch
    g = (T // pt, H // ph, W // pw)
    tok = x.reshape(C, g[0], pt, g[1], ph, g[2], pw).permute(1, 3, 5, 0, 2, 4, 6).reshape(g[0] * g[1] * g[2], C * pt * ph * pw)
    return tok, g


def unpatchify(tok: torch.Tensor, grid, out: int, patch) -> torch.Tensor:
    tg, hg, wg = grid
    pt, ph, pw = patch
    return tok.reshape(tg, hg, wg, pt, ph, pw, out).permute(6, 0, 3, 1, 4, 2, 5).reshape(out, tg * pt, hg * ph, wg * pw)


class Scail2DiT:
    def __init__(self, cfg: Scail2Config, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        w = dict(weights)
        for k in ("patch_embedding", "patch_embedding_pose", "patch_embedding_mask"):
            w[k + ".weight"] = w[k + ".weight"].reshape(cfg.dim, -1)
        self.w = nd.WeightBag(w, dtype, self.device)
        self.rope = ScailRope(cfg.head_dim)
        self._rope_cache: dict = {}

    def _heads(self, x):
        return x.view(x.shape[0], x.shape[1], self.cfg.num_heads, self.cfg.head_dim)

    def _rms(self, x, name):
        return nd.rms_norm(x, self.w[name], self.cfg.eps)

    def _block(self, x, p, e0, text_ctx, img_ctx, rope):
        cfg, w, dt = self.cfg, self.w, self.dtype
        m = w[p + ".modulation"].float() + e0                                            # [1, 6, dim]
        mod = lambda h, sc, sh: (nd.layer_norm(h, eps=cfg.eps).float() * (1 + m[:, sc:sc + 1]) + m[:, sh:sh + 1]).to(dt)   # noqa: E731
        h = mod(x, 1, 0)
        a = p + ".self_attn"
        q, k = self._heads(self._rms(w.lin(h, a + ".q"), a + ".norm_q.weight")), self._heads(self._rms(w.lin(h, a + ".k"), a + ".norm_k.weight"))
        o = nd.attention(nd.rope_interleaved(q, *rope), nd.rope_interleaved(k, *rope), self._heads(w.lin(h, a + ".v")))
        x = (x.float() + w.lin(o, a + ".o").float() * m[:, 2:3]).to(dt)
        c = p + ".cross_attn"
        hc = nd.layer_norm(x, w[p + ".norm3.weight"], w[p + ".norm3.bias"], cfg.eps)
        q = self._heads(self._rms(w.lin(hc, c + ".q"), c + ".norm_q.weight"))
        kt, vt = self._heads(self._rms(w.lin(text_ctx, c + ".k"), c + ".norm_k.weight")), self._heads(w.lin(text_ctx, c + ".v"))
        ki, vi = self._heads(self._rms(w.lin(img_ctx, c + ".k_img"), c + ".norm_k_img.weight")), self._heads(w.lin(img_ctx, c + ".v_img"))
        x = x + w.lin(nd.attention(q, kt, vt) + nd.attention(q, ki, vi), c + ".o")
        h = mod(x, 4, 3)
        f = w.lin(w.lin(h, p + ".ffn.0", act="gelu_tanh"), p + ".ffn.2")
        return (x.float() + f.float() * m[:, 5:6]).to(dt)

    def embed_text(self, context: torch.Tensor) -> torch.Tensor:
        """[L, text_dim] -> [1, text_len, dim]: zero-padded / truncated to text_len rows, then the two-layer projection."""
        L = self.cfg.text_len
        c = F.pad(context[:L], (0, 0, 0, max(0, L - context.shape[0])))[None].to(self.device, self.dtype)
        return self.w.lin(self.w.lin(c, "text_embedding.0", act="gelu_tanh"), "text_embedding.2")

    def embed_img(self, clip_fea: torch.Tensor) -> torch.Tensor:
        w, p = self.w, "img_emb.proj."
        h = nd.layer_norm(clip_fea.to(self.device, self.dtype), w[p + "0.weight"], w[p + "0.bias"], IMG_LN_EPS)
        h = w.lin(w.lin(h, p + "1", act="gelu"), p + "3")
        return nd.layer_norm(h, w[p + "4.weight"], w[p + "4.bias"], IMG_LN_EPS)

    def rope_tables(self, grid, addref: int, h_shift: int):
        key = (grid, addref, h_shift)
        if key not in self._rope_cache:
            t, h, w = grid
            parts = []
            if addref:
                parts.append(self.rope.chunk((addref, h, w), (0, h_shift, 0)))
            parts.append(self.rope.chunk((1, h, w), (addref, h_shift, 0)))
            parts.append(self.rope.chunk((t, h, w), (1 + addref, 0, 0)))
            parts.append(self.rope.chunk((t, h, w), (1 + addref, 0, self.cfg.pose_w_shift), pose_downsample=True))
            self._rope_cache = {key: tuple(torch.cat([p[i] for p in parts], 0).to(self.device) for i in (0, 1))}
        return self._rope_cache[key]

    @torch.no_grad()
    def forward(self, x, ref_latent, ref_masks, pose_latent, driving_masks, text_ctx, img_ctx, t: float, *, history_mask=None,
                additional_ref_latent=None, additional_ref_masks=None, replace_flag: bool = False) -> torch.Tensor:
        """x [16, T, H, W] noisy target; ref_latent [16, 1, H, W]; ref_masks [28, 1 + T, H, W]; pose_latent
        [16, T, H/2, W/2]; driving_masks [28, T, H/2, W/2]; text_ctx / img_ctx from embed_text / embed_img; t = sigma *
        1000 -> velocity [16, T, H, W]."""
        cfg, w, dt, dev = self.cfg, self.w, self.dtype, self.device
        ps, i2v = cfg.patch, cfg.i2v_mask_dim
        _, T, H, W = x.shape
        f32 = lambda v: v.to(dev).float()                                               # noqa: E731
        flag = lambda n, hh, ww, val: torch.full((i2v, n, hh, ww), val, device=dev)     # noqa: E731
        x20 = torch.cat([f32(x), f32(history_mask) if history_mask is not None else flag(T, H, W, 0.0)], 0)
        ref20 = torch.cat([f32(ref_latent), flag(1, H, W, 1.0)], 0)
        pose20 = torch.cat([f32(pose_latent), flag(*pose_latent.shape[1:], 1.0)], 0)
        emb = lambda lat, stem: w.lin(patchify(lat, ps)[0].to(dt), stem)               # noqa: E731
        grid = (T // ps[0], H // ps[1], W // ps[2])
        refvid = emb(torch.cat([ref20, x20], 1), "patch_embedding") + emb(f32(ref_masks), "patch_embedding_mask")
        pose = emb(pose20, "patch_embedding_pose") + emb(f32(driving_masks), "patch_embedding_mask")
        toks, addref = [], 0
        if additional_ref_latent is not None:
            if additional_ref_masks is None:
                raise ValueError("scail2: additional_ref_masks required with additional_ref_latent")
            addref = additional_ref_latent.shape[1]
            ar20 = torch.cat([f32(additional_ref_latent), flag(addref, H, W, 1.0)], 0)
            toks.append(emb(ar20, "patch_embedding") + emb(f32(additional_ref_masks), "patch_embedding_mask"))
        toks += [refvid, pose]
        rope = self.rope_tables(grid, addref, cfg.replace_h_shift if replace_flag else 0)
        h = torch.cat(toks, 0)[None]
        te = nd.sinusoidal_embedding(torch.tensor([float(t)], device=dev), cfg.freq_dim).to(dt)
        e = w.lin(w.lin(te, "time_embedding.0", act="silu"), "time_embedding.2")
        e0 = w.lin(F.silu(e.float()).to(dt), "time_projection.1").float().view(1, 6, cfg.dim)
        for i in range(cfg.num_layers):
            h = self._block(h, f"blocks.{i}", e0, text_ctx, img_ctx, rope)
        m = w["head.modulation"].float() + e.float().view(1, 1, cfg.dim)
        out = w.lin((nd.layer_norm(h, eps=cfg.eps).float() * (1 + m[:, 1:2]) + m[:, 0:1]).to(dt), "head.head")[0].float()
        ref_len, seq = grid[1] * grid[2], grid[0] * grid[1] * grid[2]
        off = (addref + 1) * ref_len
        return unpatchify(out[off:off + seq], grid, cfg.out_dim, ps)


@dataclass
class ClipVisionConfig:
    image_size: int = 224
    patch_size: int = 14
    dim: int = 1280
    num_heads: int = 16
    num_layers: int = 32
    mlp_dim: int = 5120
    eps: float = 1e-5


class ScailClip:
    """ViT-H/14 visual tower of the open-CLIP XLM-R model: the token states after all but the last block, no final norm."""

    def __init__(self, cfg: ClipVisionConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        w = dict(weights)
        w["patch_embedding.weight"] = w["patch_embedding.weight"].reshape(cfg.dim, -1)
        self.w = nd.WeightBag(w, dtype, self.device)

    @torch.no_grad()
    def encode(self, pixel: torch.Tensor) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        B, _, H, W = pixel.shape
        p = cfg.patch_size
        nh, nw = H // p, W // p
        tok = pixel.to(self.device, self.dtype).reshape(B, 3, nh, p, nw, p).permute(0, 2, 4, 1, 3, 5).reshape(B, nh * nw, 3 * p * p)
        x = torch.cat([w["cls_embedding"].expand(B, 1, -1), nd.linear(tok, w["patch_embedding.weight"])], 1) + w["pos_embedding"]
        x = nd.layer_norm(x, w["pre_norm.weight"], w["pre_norm.bias"], cfg.eps)
        hd = cfg.dim // cfg.num_heads
        for i in range(cfg.num_layers - 1):
            b = f"transformer.{i}"
            h = nd.layer_norm(x, w[b + ".norm1.weight"], w[b + ".norm1.bias"], cfg.eps)
            q, k, v = w.lin(h, b + ".attn.to_qkv").view(B, -1, 3, cfg.num_heads, hd).unbind(2)
            x = x + w.lin(nd.attention(q, k, v), b + ".attn.proj")
            h = nd.layer_norm(x, w[b + ".norm2.weight"], w[b + ".norm2.bias"], cfg.eps)
            x = x + w.lin(w.lin(h, b + ".mlp.0", act="gelu"), b + ".mlp.2")
        return x


def random_scail2_weights(cfg: Scail2Config, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    pp = cfg.patch[0] * cfg.patch[1] * cfg.patch[2]
    for name, c in (("patch_embedding", cfg.in_dim), ("patch_embedding_pose", cfg.in_dim), ("patch_embedding_mask", cfg.mask_dim)):
        w[name + ".weight"], w[name + ".bias"] = rn(cfg.dim, c, *cfg.patch) * 0.05, rn(cfg.dim) * 0.02
    lin(w, "text_embedding.0", cfg.dim, cfg.text_dim)
    lin(w, "text_embedding.2", cfg.dim, cfg.dim)
    lin(w, "time_embedding.0", cfg.dim, cfg.freq_dim)
    lin(w, "time_embedding.2", cfg.dim, cfg.dim)
    lin(w, "time_projection.1", 6 * cfg.dim, cfg.dim)
    ln = lambda p, d: w.update({p + ".weight": 1 + rn(d) * 0.05, p + ".bias": rn(d) * 0.02})      # noqa: E731
    ln("img_emb.proj.0", cfg.clip_dim)
    lin(w, "img_emb.proj.1", cfg.clip_dim, cfg.clip_dim)
    lin(w, "img_emb.proj.3", cfg.dim, cfg.clip_dim)
    ln("img_emb.proj.4", cfg.dim)
    for i in range(cfg.num_layers):
        p = f"blocks.{i}"
        w[p + ".modulation"] = rn(1, 6, cfg.dim) * 0.1
        for a, names in ((".self_attn", ("q", "k", "v", "o")), (".cross_attn", ("q", "k", "v", "o", "k_img", "v_img"))):
            for n in names:
                lin(w, p + a + "." + n, cfg.dim, cfg.dim)
            for n in ("norm_q", "norm_k") + (("norm_k_img",) if a == ".cross_attn" else ()):
                w[f"{p}{a}.{n}.weight"] = 1 + rn(cfg.dim) * 0.05
        ln(p + ".norm3", cfg.dim)
        lin(w, p + ".ffn.0", cfg.ffn_dim, cfg.dim)
        lin(w, p + ".ffn.2", cfg.dim, cfg.ffn_dim)
    w["head.modulation"] = rn(1, 2, cfg.dim) * 0.1
    lin(w, "head.head", cfg.out_dim * pp, cfg.dim)
    return w


def random_clip_weights(cfg: ClipVisionConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    n_tok = (cfg.image_size // cfg.patch_size) ** 2 + 1
    w["patch_embedding.weight"] = rn(cfg.dim, 3, cfg.patch_size, cfg.patch_size) * 0.05
    w["cls_embedding"], w["pos_embedding"] = rn(1, 1, cfg.dim) * 0.1, rn(1, n_tok, cfg.dim) * 0.1
    ln = lambda p: w.update({p + ".weight": 1 + rn(cfg.dim) * 0.05, p + ".bias": rn(cfg.dim) * 0.02})      # noqa: E731
    ln("pre_norm")
    for i in range(cfg.num_layers - 1):
        b = f"transformer.{i}"
        ln(b + ".norm1")
        ln(b + ".norm2")
        lin(w, b + ".attn.to_qkv", 3 * cfg.dim, cfg.dim)
        lin(w, b + ".attn.proj", cfg.dim, cfg.dim)
        lin(w, b + ".mlp.0", cfg.mlp_dim, cfg.dim)
        lin(w, b + ".mlp.2", cfg.dim, cfg.mlp_dim)
    return w
