"""Anima: the Cosmos-Predict2 DiT, the bundled text conditioner, and checkpoint key handling
(parity: candle-gen-anima/src/transformer.rs, conditioner.rs, rope.rs, nn.rs, vae.rs, loader.rs).

DiT (28 blocks, 16 heads of 128): latents [B, 16, T, H, W] get a zero "padding mask" channel, are cut into (1, 2, 2)
patches (17 * 4 features, ordered channel-major) and embedded by a linear. Each block has three gated residual
branches (self-attention with rotary, cross-attention into the text states, GELU MLP); each branch's shift / scale / gate
is a two-layer low-rank projection (2048 -> 256 -> 3 * 2048) of SiLU(normed sinusoid) plus the timestep MLP's output.
q / k are RMS-normed per head. Rotary is half-rotation over a head split into (time 44, row 42, column 42) wide axes
with NTK-scaled bases (scales 1, 4, 4). The network's time input is sigma itself.

Conditioner: an embedding over T5 token ids is refined by 6 blocks (self-attention, cross-attention into the masked
Qwen3 states, GELU MLP; RMS pre-norms, q / k norms, rotary on both sides by position), projected, normed and
right-padded with zeros to 512 rows.

One implementation for both backends (nn_dual)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

QK_EPS, NORM_EPS = 1e-5, 1e-6
PREFIX_ANCHOR = ".x_embedder.proj.1.weight"


@dataclass
class CosmosConfig:
    in_channels: int = 16
    out_channels: int = 16
    num_attention_heads: int = 16
    attention_head_dim: int = 128
    num_layers: int = 28
    mlp_ratio: float = 4.0
    text_embed_dim: int = 1024
    adaln_lora_dim: int = 256
    max_size: tuple[int, int, int] = (128, 120, 120)
    patch_size: tuple[int, int, int] = (1, 2, 2)
    rope_scale: tuple[float, float, float] = (1.0, 4.0, 4.0)
    concat_padding_mask: bool = True

    @property
    def hidden(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @staticmethod
    def from_json(j: dict) -> "CosmosConfig":
        d = {k: (tuple(j[k]) if isinstance(j[k], list) else j[k]) for k in CosmosConfig.__dataclass_fields__ if k in j}
        return CosmosConfig(**d)


@dataclass
class ConditionerConfig:
    source_dim: int = 1024
    target_dim: int = 1024
    model_dim: int = 1024
    num_layers: int = 6
    num_attention_heads: int = 16
    mlp_ratio: float = 4.0
    target_vocab_size: int = 32128
    min_sequence_length: int = 512
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.model_dim // self.num_attention_heads

    @staticmethod
    def from_json(j: dict) -> "ConditionerConfig":
        return ConditionerConfig(**{k: j[k] for k in ConditionerConfig.__dataclass_fields__ if k in j})


def random_anima_weights(cfg: CosmosConfig, ccfg: ConditionerConfig, seed: int = 0, std: float = 0.05) -> dict[str, torch.Tensor]:
    """DiT keys at the root, conditioner keys under `llm_adapter.` (the checkpoint adds a root prefix to both)."""
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    H, hd, r = cfg.hidden, cfg.attention_head_dim, cfg.adaln_lora_dim
    pin = (cfg.in_channels + (1 if cfg.concat_padding_mask else 0)) * cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2]
    lin(w, "x_embedder.proj.1", H, pin, std, bias=False)
    lin(w, "t_embedder.1.linear_1", H, H, std, bias=False)
    lin(w, "t_embedder.1.linear_2", 3 * H, H, std, bias=False)
    w["t_embedding_norm.weight"] = 1.0 + rn(H) * 0.1
    for i in range(cfg.num_layers):
        b = f"blocks.{i}"
        for n in ("self_attn", "cross_attn", "mlp"):
            lin(w, f"{b}.adaln_modulation_{n}.1", r, H, std, bias=False)
            lin(w, f"{b}.adaln_modulation_{n}.2", 3 * H, r, std, bias=False)
        for a, kv in (("self_attn", H), ("cross_attn", cfg.text_embed_dim)):
            lin(w, f"{b}.{a}.q_proj", H, H, std, bias=False)
            lin(w, f"{b}.{a}.k_proj", H, kv, std, bias=False)
            lin(w, f"{b}.{a}.v_proj", H, kv, std, bias=False)
            lin(w, f"{b}.{a}.output_proj", H, H, std, bias=False)
            w[f"{b}.{a}.q_norm.weight"], w[f"{b}.{a}.k_norm.weight"] = 1.0 + rn(hd) * 0.1, 1.0 + rn(hd) * 0.1
        lin(w, b + ".mlp.layer1", int(H * cfg.mlp_ratio), H, std, bias=False)
        lin(w, b + ".mlp.layer2", H, int(H * cfg.mlp_ratio), std, bias=False)
    lin(w, "final_layer.adaln_modulation.1", r, H, std, bias=False)
    lin(w, "final_layer.adaln_modulation.2", 2 * H, r, std, bias=False)
    lin(w, "final_layer.linear", cfg.out_channels * cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2], H, std, bias=False)
    M, chd = ccfg.model_dim, ccfg.head_dim
    c = "llm_adapter."
    w[c + "embed.weight"] = rn(ccfg.target_vocab_size, M) * 0.3
    for i in range(ccfg.num_layers):
        b = f"{c}blocks.{i}"
        for n in ("norm_self_attn", "norm_cross_attn", "norm_mlp"):
            w[f"{b}.{n}.weight"] = 1.0 + rn(M) * 0.1
        for a, kv in (("self_attn", M), ("cross_attn", ccfg.source_dim)):
            lin(w, f"{b}.{a}.q_proj", M, M, std, bias=False)
            lin(w, f"{b}.{a}.k_proj", M, kv, std, bias=False)
            lin(w, f"{b}.{a}.v_proj", M, kv, std, bias=False)
            lin(w, f"{b}.{a}.o_proj", M, M, std, bias=False)
            w[f"{b}.{a}.q_norm.weight"], w[f"{b}.{a}.k_norm.weight"] = 1.0 + rn(chd) * 0.1, 1.0 + rn(chd) * 0.1
        lin(w, b + ".mlp.0", int(M * ccfg.mlp_ratio), M, std)
        lin(w, b + ".mlp.2", M, int(M * ccfg.mlp_ratio), std)
    lin(w, c + "out_proj", ccfg.target_dim, M, std)
    w[c + "norm.weight"] = 1.0 + rn(ccfg.target_dim) * 0.1
    return w


def detect_dit_prefix(keys) -> str:
    """The checkpoint's root prefix (`net`, `model.diffusion_model`, ...) from the one key every file has."""
    for k in keys:
        if k.endswith(PREFIX_ANCHOR) and "llm_adapter" not in k:
            return k[: -len(PREFIX_ANCHOR)]
    raise ValueError(f"no key ending in {PREFIX_ANCHOR}: not an Anima DiT checkpoint")


def cosmos_rope(cfg: CosmosConfig, pe_t: int, pe_h: int, pe_w: int):
    """cos, sin [S, head_dim / 2] in half-rotation layout (the first half of the head pairs with the second)."""
    mt, mh, mw = cfg.max_size
    if pe_t > mt or pe_h > mh or pe_w > mw:
        raise ValueError(f"latent grid (t={pe_t}, h={pe_h}, w={pe_w}) exceeds the rotary tables' limits {cfg.max_size}")
    hd = cfg.attention_head_dim
    dh = dw = hd // 6 * 2
    dt = hd - dh - dw

    def freqs(scale, dim):
        theta = 10000.0 * scale ** (dim / (dim - 2.0))
        return theta ** (-torch.arange(0, dim, 2, dtype=torch.float64) / dim)

    t, h, w = torch.meshgrid(torch.arange(pe_t, dtype=torch.float64), torch.arange(pe_h, dtype=torch.float64),
                             torch.arange(pe_w, dtype=torch.float64), indexing="ij")
    ang = torch.cat([t.reshape(-1, 1) * freqs(cfg.rope_scale[0], dt)[None], h.reshape(-1, 1) * freqs(cfg.rope_scale[1], dh)[None],
                     w.reshape(-1, 1) * freqs(cfg.rope_scale[2], dw)[None]], dim=1)
    return ang.cos().float(), ang.sin().float()


def _text_rope(n: int, dim: int, theta: float):
    ang = torch.arange(n, dtype=torch.float64)[:, None] * theta ** (-torch.arange(0, dim, 2, dtype=torch.float64) / dim)[None]
    return ang.cos().float(), ang.sin().float()


class CosmosDiT:
    def __init__(self, cfg: CosmosConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.bag = nd.WeightBag({k: v for k, v in weights.items() if not k.startswith("llm_adapter.")}, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device
        self._rope = None

    def weight_bytes(self) -> int:
        return self.bag.nbytes()

    def _attn(self, x, ctx, p, rope):
        cfg = self.cfg
        B, S, _ = x.shape
        nh, hd = cfg.num_attention_heads, cfg.attention_head_dim
        src = x if ctx is None else ctx
        q = nd.rms_norm(self.bag.lin(x, p + ".q_proj").reshape(B, S, nh, hd), self.bag[p + ".q_norm.weight"], QK_EPS)
        k = nd.rms_norm(self.bag.lin(src, p + ".k_proj").reshape(B, -1, nh, hd), self.bag[p + ".k_norm.weight"], QK_EPS)
        v = self.bag.lin(src, p + ".v_proj").reshape(B, -1, nh, hd)
        if rope is not None:
            q, k = nd.rope_half(q, *rope), nd.rope_half(k, *rope)
        return self.bag.lin(nd.attention(q, k, v), p + ".output_proj")

    def forward_grad(self, latents: torch.Tensor, sigma: torch.Tensor, encoder: torch.Tensor) -> torch.Tensor:
        """latents [B, C, T, H, W], sigma [B], encoder [B, L, text_embed_dim] -> velocity [B, C, T, H, W] (fp32)."""
        cfg, dt, dev = self.cfg, self.dtype, self.device
        x = latents.to(dev, dt)
        B, C, T, Hl, Wl = x.shape
        pt, ph, pw = cfg.patch_size
        et, eh, ew = T // pt, Hl // ph, Wl // pw
        if cfg.concat_padding_mask:
            x = torch.cat([x, torch.zeros(B, 1, T, Hl, Wl, device=dev, dtype=dt)], dim=1)
        Ci = x.shape[1]
        tok = x.reshape(B, Ci, et, pt, eh, ph, ew, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, et * eh * ew, Ci * pt * ph * pw)
        if self._rope is None or self._rope[0] != (et, eh, ew):
            c, s = cosmos_rope(cfg, et, eh, ew)
            self._rope = ((et, eh, ew), c.to(dev), s.to(dev))
        rope = self._rope[1:]
        h = self.bag.lin(tok, "x_embedder.proj.1")
        proj = nd.sinusoidal_embedding(sigma.to(dev), cfg.hidden).to(dt)
        temb = self.bag.lin(self.bag.lin(proj, "t_embedder.1.linear_1", act="silu"), "t_embedder.1.linear_2")       # [B, 3H]
        emb = F.silu(nd.rms_norm(proj, self.bag["t_embedding_norm.weight"], NORM_EPS).float()).to(dt)
        enc = encoder.to(dev, dt)

        def mod(name, n):
            e = self.bag.lin(self.bag.lin(emb, name + ".1"), name + ".2") + temb[:, : n * cfg.hidden]
            return [c[:, None, :] for c in e.chunk(n, dim=-1)]

        for i in range(cfg.num_layers):
            b = f"blocks.{i}"
            sh, sc, g = mod(b + ".adaln_modulation_self_attn", 3)
            h = h + g * self._attn(nd.layer_norm(h, eps=NORM_EPS) * (1 + sc) + sh, None, b + ".self_attn", rope)
            sh, sc, g = mod(b + ".adaln_modulation_cross_attn", 3)
            h = h + g * self._attn(nd.layer_norm(h, eps=NORM_EPS) * (1 + sc) + sh, enc, b + ".cross_attn", None)
            sh, sc, g = mod(b + ".adaln_modulation_mlp", 3)
            m = self.bag.lin(nd.layer_norm(h, eps=NORM_EPS) * (1 + sc) + sh, b + ".mlp.layer1", act="gelu")
            h = h + g * self.bag.lin(m, b + ".mlp.layer2")
        sh, sc = mod("final_layer.adaln_modulation", 2)
        out = self.bag.lin(nd.layer_norm(h, eps=NORM_EPS) * (1 + sc) + sh, "final_layer.linear").float()
        oc = cfg.out_channels
        return out.reshape(B, et, eh, ew, ph, pw, pt, oc).permute(0, 7, 1, 6, 2, 4, 3, 5).reshape(B, oc, et * pt, eh * ph, ew * pw)

    @torch.no_grad()
    def forward(self, latents, sigma, encoder):
        return self.forward_grad(latents, sigma, encoder)


class AnimaTextConditioner:
    def __init__(self, cfg: ConditionerConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        pre = "llm_adapter."
        self.bag = nd.WeightBag({k[len(pre):]: v for k, v in weights.items() if k.startswith(pre)}, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device

    def _attn(self, x, ctx, p, q_rope, k_rope):
        cfg = self.cfg
        B, S, _ = x.shape
        nh, hd = cfg.num_attention_heads, cfg.head_dim
        src = x if ctx is None else ctx
        q = nd.rms_norm(self.bag.lin(x, p + ".q_proj").reshape(B, S, nh, hd), self.bag[p + ".q_norm.weight"], cfg.norm_eps)
        k = nd.rms_norm(self.bag.lin(src, p + ".k_proj").reshape(B, -1, nh, hd), self.bag[p + ".k_norm.weight"], cfg.norm_eps)
        v = self.bag.lin(src, p + ".v_proj").reshape(B, -1, nh, hd)
        return self.bag.lin(nd.attention(nd.rope_half(q, *q_rope), nd.rope_half(k, *k_rope), v), p + ".o_proj")

    @torch.no_grad()
    def forward(self, source_hidden: torch.Tensor, target_ids: torch.Tensor) -> torch.Tensor:
        """source [B, Ss, source_dim] (masked language-model states), target ids [B, St] -> [B, max(St, 512), target_dim]."""
        cfg, dev, dt = self.cfg, self.device, self.dtype
        src = source_hidden.to(dev, dt)
        ids = target_ids.to(dev)
        h = self.bag["embed.weight"][ids]
        St, Ss = ids.shape[1], src.shape[1]
        tr = tuple(t.to(dev) for t in _text_rope(St, cfg.head_dim, cfg.rope_theta))
        sr = tuple(t.to(dev) for t in _text_rope(Ss, cfg.head_dim, cfg.rope_theta))
        for i in range(cfg.num_layers):
            b = f"blocks.{i}"
            h = h + self._attn(nd.rms_norm(h, self.bag[b + ".norm_self_attn.weight"], cfg.norm_eps), None, b + ".self_attn", tr, tr)
            h = h + self._attn(nd.rms_norm(h, self.bag[b + ".norm_cross_attn.weight"], cfg.norm_eps), src, b + ".cross_attn", tr, sr)
            m = self.bag.lin(nd.rms_norm(h, self.bag[b + ".norm_mlp.weight"], cfg.norm_eps), b + ".mlp.0", act="gelu")
            h = h + self.bag.lin(m, b + ".mlp.2")
        h = nd.rms_norm(self.bag.lin(h, "out_proj"), self.bag["norm.weight"], cfg.norm_eps)
        if St < cfg.min_sequence_length:
            h = torch.cat([h, torch.zeros(h.shape[0], cfg.min_sequence_length - St, h.shape[2], device=dev, dtype=dt)], dim=1)
        return h


# ---- autoencoder checkpoint keys --------------------------------------------------------------------------------------
def _residual(k: str) -> str:
    for a, b in ((".residual.0.", ".norm1."), (".residual.2.", ".conv1."), (".residual.3.", ".norm2."),
                 (".residual.6.", ".conv2."), (".shortcut.", ".conv_shortcut.")):
        k = k.replace(a, b)
    return k


def convert_vae_key(k: str) -> str:
    """Original (Wan-style) autoencoder key -> the diffusers spelling the Qwen-Image decoder reads."""
    simple = (("conv1.", "quant_conv."), ("conv2.", "post_quant_conv."), ("encoder.conv1.", "encoder.conv_in."),
              ("decoder.conv1.", "decoder.conv_in."), ("encoder.head.0.", "encoder.norm_out."),
              ("encoder.head.2.", "encoder.conv_out."), ("decoder.head.0.", "decoder.norm_out."),
              ("decoder.head.2.", "decoder.conv_out."))
    for a, b in simple:
        if k.startswith(a):
            return b + k[len(a):]
    if k.startswith("encoder.downsamples."):
        return _residual("encoder.down_blocks." + k[len("encoder.downsamples."):])
    if k.startswith("decoder.upsamples."):
        idx, _, rest = k[len("decoder.upsamples."):].partition(".")
        i = int(idx)
        if i in (3, 7, 11):
            return _residual(f"decoder.up_blocks.{(i - 3) // 4}.upsamplers.0.{rest}")
        return _residual(f"decoder.up_blocks.{i // 4}.resnets.{i % 4}.{rest}")
    if k.startswith(("encoder.middle.", "decoder.middle.")):
        for a, b in ((".middle.0.", ".mid_block.resnets.0."), (".middle.1.", ".mid_block.attentions.0."),
                     (".middle.2.", ".mid_block.resnets.1.")):
            k = k.replace(a, b)
    return _residual(k)


def anima_sigmas(steps: int, shift: float = 3.0) -> list[float]:
    n = max(1, steps)
    out = []
    for i in range(n):
        s = 1.0 if n == 1 else 1.0 + i * (1.0 / n - 1.0) / (n - 1)
        out.append(shift * s / (1.0 + (shift - 1.0) * s))
    return out + [0.0]
