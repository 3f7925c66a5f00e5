"""Boogu-Image hybrid MMDiT (parity: candle-gen-boogu/src/transformer/{mod,block,rope}.rs, config.rs; checkpoint keys
are the diffusers names of the published transformer).

A Lumina-Image-2 / OmniGen2-lineage network: the instruction states (last hidden layer of a Qwen3-VL language tower)
are RMS-normalised and projected, then refined by two unmodulated blocks; the 2x2-patched 16-channel latent is embedded
and refined by two timestep-modulated blocks; reference images (edit) go through their own patch embedder, an image
index embedding and their own refiner, and are laid in front of the noisy image tokens. Eight double-stream layers
(joint attention of the two streams with separate projections, one extra image-only self-attention, separate SwiGLU
MLPs) are followed by 32 single-stream layers over [instruction, references, image]. Every residual branch is
RMS-normalised after the op and gated by tanh of a timestep projection; attention is grouped-query (28 / 7 heads of
120) with per-head q / k RMSNorm and a three-axis adjacent-pair rotary position: instruction token i sits at (i, i, i),
an image grid at (t, row, column) with t = instruction length (+ the larger side of every earlier reference grid).

One implementation for both backends (nn_dual): fp32 oracle on CPU; bf16 with the tcgen05 GEMM / attention kernels on
a CUDA device (120-wide heads are zero-padded onto the 128-wide attention kernel)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd

QK_EPS = 1e-5


@dataclass
class BooguConfig:
    patch_size: int = 2
    in_channels: int = 16
    out_channels: int = 16
    hidden_size: int = 3360
    num_layers: int = 40
    num_double_stream_layers: int = 8
    num_refiner_layers: int = 2
    num_attention_heads: int = 28
    num_kv_heads: int = 7
    norm_eps: float = 1e-5
    axes_dim_rope: tuple = (40, 40, 40)
    rope_theta: float = 10000.0
    reduce_type: str = "mean"
    timestep_scale: float = 1000.0
    text_dim: int = 4096
    multiple_of: int = 256
    ffn_dim_multiplier: float | None = None

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def num_single_stream_layers(self) -> int:
        return self.num_layers - self.num_double_stream_layers

    @staticmethod
    def from_json(j: dict) -> "BooguConfig":
        c = BooguConfig()
        for k in ("patch_size", "in_channels", "hidden_size", "num_layers", "num_double_stream_layers", "num_refiner_layers",
                  "num_attention_heads", "num_kv_heads", "norm_eps", "timestep_scale", "multiple_of", "ffn_dim_multiplier"):
            if j.get(k) is not None:
                setattr(c, k, j[k])
        c.out_channels = j.get("out_channels") or c.in_channels
        if isinstance(j.get("axes_dim_rope"), list) and len(j["axes_dim_rope"]) == 3:
            c.axes_dim_rope = tuple(int(v) for v in j["axes_dim_rope"])
        c.reduce_type = (j.get("instruction_feature_configs") or {}).get("reduce_type", c.reduce_type)
        c.text_dim = j.get("instruction_feat_dim", j.get("text_dim", c.text_dim))
        c.validate()
        return c

    def validate(self) -> None:
        if self.head_dim != sum(self.axes_dim_rope):
            raise ValueError(f"boogu: head_dim ({self.head_dim}) must equal sum(axes_dim_rope) ({sum(self.axes_dim_rope)})")
        if self.num_double_stream_layers > self.num_layers:
            raise ValueError(f"boogu: num_double_stream_layers ({self.num_double_stream_layers}) > num_layers ({self.num_layers})")
        if self.num_attention_heads % self.num_kv_heads:
            raise ValueError(f"boogu: num_attention_heads ({self.num_attention_heads}) not divisible by num_kv_heads "
                             f"({self.num_kv_heads})")
        if self.reduce_type != "mean":
            raise ValueError(f"boogu: unsupported instruction reduce_type {self.reduce_type!r} (only \"mean\")")


def rope_positions(cap_len: int, ref_grids: list[tuple[int, int]], ht: int, wt: int) -> torch.Tensor:
    """[cap + refs + image, 3] float positions in token order."""
    idx = torch.arange(cap_len, dtype=torch.float32)
    rows = [torch.stack([idx, idx, idx], 1)]
    shift = cap_len
    for h, w in list(ref_grids) + [(ht, wt)]:
        g = torch.zeros(h, w, 3)
        g[..., 0] = float(shift)
        g[..., 1] = torch.arange(h, dtype=torch.float32)[:, None]
        g[..., 2] = torch.arange(w, dtype=torch.float32)[None, :]
        rows.append(g.reshape(-1, 3))
        shift += max(h, w)
    return torch.cat(rows, 0)


class BooguDiT:
    def __init__(self, cfg: BooguConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        self.w = nd.WeightBag(weights, dtype, self.device)
        self._rope: dict = {}

    # ---- pieces -----------------------------------------------------------------------------------------------------------
    def _rms(self, x, name, eps=None):
        return nd.rms_norm(x, self.w[name], self.cfg.norm_eps if eps is None else eps)

    def _self_attn(self, x, p, rope):
        cfg = self.cfg
        B, S, _ = x.shape
        H, K, D = cfg.num_attention_heads, cfg.num_kv_heads, cfg.head_dim
        w = self.w
        q = self._rms(w.lin(x, p + ".to_q").view(B, S, H, D), p + ".norm_q.weight", QK_EPS)
        k = self._rms(w.lin(x, p + ".to_k").view(B, S, K, D), p + ".norm_k.weight", QK_EPS)
        v = w.lin(x, p + ".to_v").view(B, S, K, D)
        o = nd.attention(nd.rope_interleaved(q, *rope), nd.rope_interleaved(k, *rope), v)
        return w.lin(o, p + ".to_out.0")

    def _joint_attn(self, img, ins, p, rope):
        cfg, w = self.cfg, self.w
        B, Li, _ = img.shape
        Lt = ins.shape[1]
        H, K, D = cfg.num_attention_heads, cfg.num_kv_heads, cfg.head_dim
        cat = lambda n, heads: torch.cat([w.lin(ins, f"{p}.processor.instruct_to_{n}").view(B, Lt, heads, D),       # noqa: E731
                                          w.lin(img, f"{p}.processor.img_to_{n}").view(B, Li, heads, D)], 1)
        q = self._rms(cat("q", H), p + ".norm_q.weight", QK_EPS)
        k = self._rms(cat("k", K), p + ".norm_k.weight", QK_EPS)
        o = nd.attention(nd.rope_interleaved(q, *rope), nd.rope_interleaved(k, *rope), cat("v", K))
        merged = torch.cat([w.lin(o[:, :Lt], p + ".processor.instruct_out"), w.lin(o[:, Lt:], p + ".processor.img_out")], 1)
        return w.lin(merged, p + ".to_out.0")

    def _swiglu(self, x, p):
        w = self.w
        return w.lin((F.silu(w.lin(x, p + ".linear_1").float()) * w.lin(x, p + ".linear_3").float()).to(x.dtype), p + ".linear_2")

    def _modnorm(self, x, temb_act, p):
        """-> (rmsnorm(x) * (1 + a), b, c, d) with (a, b, c, d) = the four chunks of linear(silu(temb))."""
        a, b, c, d = self.w.lin(temb_act, p + ".linear").float().chunk(4, -1)
        return (self._rms(x, p + ".norm.weight").float() * (1 + a)).to(x.dtype), b, c, d

    def _gated(self, x, gate, branch, norm):
        return (x.float() + torch.tanh(gate) * self._rms(branch, norm).float()).to(x.dtype)

    def _plain_block(self, x, p, rope):
        x = x + self._rms(self._self_attn(self._rms(x, p + ".norm1.weight"), p + ".attn", rope), p + ".norm2.weight")
        return x + self._rms(self._swiglu(self._rms(x, p + ".ffn_norm1.weight"), p + ".feed_forward"), p + ".ffn_norm2.weight")

    def _mod_block(self, x, p, rope, ta):
        n, gate_msa, scale_mlp, gate_mlp = self._modnorm(x, ta, p + ".norm1")
        x = self._gated(x, gate_msa, self._self_attn(n, p + ".attn", rope), p + ".norm2.weight")
        h = (self._rms(x, p + ".ffn_norm1.weight").float() * (1 + scale_mlp)).to(x.dtype)
        return self._gated(x, gate_mlp, self._swiglu(h, p + ".feed_forward"), p + ".ffn_norm2.weight")

    def _double_block(self, img, ins, p, joint_rope, img_rope, ta):
        Lt = ins.shape[1]
        i1, i_gate_msa, i_scale_mlp, i_gate_mlp = self._modnorm(img, ta, p + ".img_norm1")
        i2, i_shift_mlp, _, _ = self._modnorm(img, ta, p + ".img_norm2")
        i3, i_gate_self, _, _ = self._modnorm(img, ta, p + ".img_norm3")
        t1, t_gate_msa, t_scale_mlp, t_gate_mlp = self._modnorm(ins, ta, p + ".instruct_norm1")
        t2, t_shift_mlp, _, _ = self._modnorm(ins, ta, p + ".instruct_norm2")
        joint = self._joint_attn(i1, t1, p + ".img_instruct_attn", joint_rope)
        img_self = self._self_attn(i3, p + ".img_self_attn", img_rope)
        img = self._gated(img, i_gate_msa, joint[:, Lt:], p + ".img_attn_norm.weight")
        img = self._gated(img, i_gate_self, img_self, p + ".img_self_attn_norm.weight")
        h = (i2.float() * (1 + i_scale_mlp) + i_shift_mlp).to(img.dtype)
        img = self._gated(img, i_gate_mlp, self._swiglu(self._rms(h, p + ".img_ffn_norm1.weight"), p + ".img_feed_forward"),
                          p + ".img_ffn_norm2.weight")
        ins = self._gated(ins, t_gate_msa, joint[:, :Lt], p + ".instruct_attn_norm.weight")
        h = (t2.float() * (1 + t_scale_mlp) + t_shift_mlp).to(ins.dtype)
        ins = self._gated(ins, t_gate_mlp, self._swiglu(self._rms(h, p + ".instruct_ffn_norm1.weight"), p + ".instruct_feed_forward"),
                          p + ".instruct_ffn_norm2.weight")
        return img, ins

    def patchify(self, z):
        """[B, C, H, W] -> [B, (H/p)(W/p), p*p*C] with a patch ordered (row, column, channel)."""
        B, C, H, W = z.shape
        p = self.cfg.patch_size
        return z.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(B, (H // p) * (W // p), p * p * C)

    def unpatchify(self, x, ht, wt):
        B, p = x.shape[0], self.cfg.patch_size
        return x.reshape(B, ht, wt, p, p, -1).permute(0, 5, 1, 3, 2, 4).reshape(B, -1, ht * p, wt * p)

    def _rope_tables(self, cap_len, ref_grids, ht, wt):
        key = (cap_len, tuple(ref_grids), ht, wt)
        if key not in self._rope:
            if len(self._rope) >= 4:
                self._rope.pop(next(iter(self._rope)))
            cos, sin = nd.axis_rope_tables(rope_positions(cap_len, ref_grids, ht, wt), self.cfg.axes_dim_rope, self.cfg.rope_theta)
            self._rope[key] = (cos.to(self.device), sin.to(self.device))
        return self._rope[key]

    # ---- forward ----------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, latent, timestep, instruction, ref_latents=()):
        """latent [1, C, H, W]; timestep [1] in [0, 1] (0 = noise, 1 = data); instruction [1, L, text_dim]; ref_latents:
        clean reference latents [1, C, h, w] (edit) -> the velocity towards the data [1, C, H, W]."""
        cfg, w, dt, dev = self.cfg, self.w, self.dtype, self.device
        p = cfg.patch_size
        _, _, H, W = latent.shape
        ht, wt = H // p, W // p
        n_img = ht * wt
        ins = instruction.to(dev, dt)
        cap = ins.shape[1]
        te = nd.sinusoidal_embedding(timestep.to(dev).float() * cfg.timestep_scale, 256).to(dt)
        tp = "time_caption_embed."
        temb = w.lin(w.lin(te, tp + "timestep_embedder.linear_1", act="silu"), tp + "timestep_embedder.linear_2")[:, None]
        ta = F.silu(temb.float()).to(dt)
        ins = w.lin(self._rms(ins, tp + "caption_embedder.0.weight"), tp + "caption_embedder.1")
        img = w.lin(self.patchify(latent.to(dev, dt)), "x_embedder")
        refs, grids = [], []
        for j, rl in enumerate(ref_latents):
            r = w.lin(self.patchify(rl.to(dev, dt)), "ref_image_patch_embedder") + w["image_index_embedding"][j].view(1, 1, -1)
            refs.append(r)
            grids.append((rl.shape[2] // p, rl.shape[3] // p))
        cos, sin = self._rope_tables(cap, grids, ht, wt)
        n_ref = sum(h * w_ for h, w_ in grids)
        sl = lambda a, b: (cos[a:b], sin[a:b])                        # noqa: E731
        total = cap + n_ref + n_img
        for i in range(cfg.num_refiner_layers):
            ins = self._plain_block(ins, f"context_refiner.{i}", sl(0, cap))
        for i in range(cfg.num_refiner_layers):
            img = self._mod_block(img, f"noise_refiner.{i}", sl(cap + n_ref, total), ta)
        if refs:
            at, done = cap, []
            for r in refs:
                for i in range(cfg.num_refiner_layers):
                    r = self._mod_block(r, f"ref_image_refiner.{i}", sl(at, at + r.shape[1]), ta)
                done.append(r)
                at += r.shape[1]
            img = torch.cat(done + [img], 1)
        for i in range(cfg.num_double_stream_layers):
            img, ins = self._double_block(img, ins, f"double_stream_layers.{i}", (cos, sin), sl(cap, total), ta)
        x = torch.cat([ins, img], 1)
        for i in range(cfg.num_single_stream_layers):
            x = self._mod_block(x, f"single_stream_layers.{i}", (cos, sin), ta)
        scale = w.lin(ta, "norm_out.linear_1").float()
        x = (nd.layer_norm(x, eps=1e-6).float() * (1 + scale)).to(dt)
        return self.unpatchify(w.lin(x[:, -n_img:], "norm_out.linear_2").float(), ht, wt)


def ffn_dim(cfg: BooguConfig) -> int:
    d = int(cfg.hidden_size / 3 * 8)
    if cfg.ffn_dim_multiplier is not None:
        d = int(cfg.ffn_dim_multiplier * d)
    return cfg.multiple_of * ((d + cfg.multiple_of - 1) // cfg.multiple_of)


def random_boogu_weights(cfg: BooguConfig, seed: int = 0, max_refs: int = 5) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed)
    w: dict[str, torch.Tensor] = {}
    D, hd, H, K = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_kv_heads
    T, ff, pd = min(D, 1024), ffn_dim(cfg), cfg.patch_size ** 2 * cfg.in_channels
    norm = lambda n, d=D: w.__setitem__(n, 1 + rn(d) * 0.05)                # noqa: E731

    def attn(p):
        lin(w, p + ".to_q", H * hd, D, bias=False)
        lin(w, p + ".to_k", K * hd, D, bias=False)
        lin(w, p + ".to_v", K * hd, D, bias=False)
        lin(w, p + ".to_out.0", D, H * hd, bias=False)
        norm(p + ".norm_q.weight", hd)
        norm(p + ".norm_k.weight", hd)

    def swiglu(p):
        lin(w, p + ".linear_1", ff, D, bias=False)
        lin(w, p + ".linear_3", ff, D, bias=False)
        lin(w, p + ".linear_2", D, ff, bias=False)

    def modnorm(p):
        lin(w, p + ".linear", 4 * D, T)
        norm(p + ".norm.weight")

    def block(p, modulated):
        attn(p + ".attn")
        swiglu(p + ".feed_forward")
        modnorm(p + ".norm1") if modulated else norm(p + ".norm1.weight")
        for n in ("norm2", "ffn_norm1", "ffn_norm2"):
            norm(f"{p}.{n}.weight")

    lin(w, "x_embedder", D, pd)
    lin(w, "ref_image_patch_embedder", D, pd)
    w["image_index_embedding"] = rn(max_refs, D) * 0.05
    norm("time_caption_embed.caption_embedder.0.weight", cfg.text_dim)
    lin(w, "time_caption_embed.caption_embedder.1", D, cfg.text_dim)
    lin(w, "time_caption_embed.timestep_embedder.linear_1", T, 256)
    lin(w, "time_caption_embed.timestep_embedder.linear_2", T, T)
    for i in range(cfg.num_refiner_layers):
        block(f"context_refiner.{i}", False)
        block(f"noise_refiner.{i}", True)
        block(f"ref_image_refiner.{i}", True)
    for i in range(cfg.num_double_stream_layers):
        p = f"double_stream_layers.{i}"
        for n in ("q", "k", "v"):
            heads = H if n == "q" else K
            lin(w, f"{p}.img_instruct_attn.processor.img_to_{n}", heads * hd, D, bias=False)
            lin(w, f"{p}.img_instruct_attn.processor.instruct_to_{n}", heads * hd, D, bias=False)
        lin(w, p + ".img_instruct_attn.processor.img_out", D, H * hd, bias=False)
        lin(w, p + ".img_instruct_attn.processor.instruct_out", D, H * hd, bias=False)
        lin(w, p + ".img_instruct_attn.to_out.0", D, D, bias=False)
        norm(p + ".img_instruct_attn.norm_q.weight", hd)
        norm(p + ".img_instruct_attn.norm_k.weight", hd)
        attn(p + ".img_self_attn")
        swiglu(p + ".img_feed_forward")
        swiglu(p + ".instruct_feed_forward")
        for n in ("img_norm1", "img_norm2", "img_norm3", "instruct_norm1", "instruct_norm2"):
            modnorm(f"{p}.{n}")
        for n in ("img_attn_norm", "img_self_attn_norm", "img_ffn_norm1", "img_ffn_norm2", "instruct_attn_norm",
                  "instruct_ffn_norm1", "instruct_ffn_norm2"):
            norm(f"{p}.{n}.weight")
    for i in range(cfg.num_single_stream_layers):
        block(f"single_stream_layers.{i}", True)
    lin(w, "norm_out.linear_1", D, T)
    lin(w, "norm_out.linear_2", cfg.patch_size ** 2 * cfg.out_channels, D)
    return w
