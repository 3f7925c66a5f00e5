"""Krea 2 dense single-stream DiT (parity: candle-gen-krea/src/transformer/{mod,block,rope}.rs, config.rs; checkpoint
keys are the diffusers `Krea2Transformer2DModel` names).

The prompt arrives as a stack of `num_text_layers` hidden layers of the condition encoder per token
([B, L, 12, 2560]). `text_fusion` turns it into one stream: gated-attention blocks run ACROSS the layer axis (every
token is a sequence of 12 layer states), a bias-free Linear(12 -> 1) collapses that axis, more blocks run over the
token axis; `txt_in` (RMS scale + 2-layer GELU MLP) lifts it to the model width. Image latents are 2 x 2 patchified
(channel-major) and embedded by `img_in`. [text, image] then runs through `num_layers` single-stream blocks:

    m = time_mod_proj(gelu(t)) + scale_shift_table           -> pre / post {scale, shift, gate}
    x += pregate  * attn(rms(x) * (1 + prescale)  + preshift)
    x += postgate * swiglu(rms(x) * (1 + postscale) + postshift)

Attention is grouped-query (48 / 12 heads of 128) with per-head RMS scale on q and k, interleaved three-axis rotary
embedding (text at the origin, image tokens at (0, row, column), reference images of an edit at frame 1, 2, ...), and
an output gate: out = to_out(sdpa * sigmoid(to_gate(x))). "RMS scale" stores `scale` with the weight `scale + 1`.

One implementation serves both backends (see nn_dual): fp32 on the CPU oracle backend; bf16 on a CUDA device with every
projection on the tcgen05 GEMM and attention on the tcgen05 flash-attention kernel (grouped-query heads natively).
On the device the q / k / v / gate projections of a block run as ONE GEMM over a concatenated weight, and the SwiGLU
gate / up pair as one GEMM; `quantize_nvfp4()` repacks the block projections to NVFP4 (W4A16 or W4A4)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import nn_dual as nd


@dataclass
class KreaConfig:
    in_channels: int = 64
    patch_size: int = 2
    num_attention_heads: int = 48
    num_kv_heads: int = 12
    attention_head_dim: int = 128
    num_layers: int = 28
    intermediate_size: int = 16384
    norm_eps: float = 1e-5
    axes_dims_rope: tuple[int, int, int] = (32, 48, 48)
    rope_theta: float = 1000.0
    timestep_embed_dim: int = 256
    num_text_layers: int = 12
    num_layerwise_text_blocks: int = 2
    num_refiner_text_blocks: int = 2
    text_hidden_dim: int = 2560
    text_intermediate_size: int = 6912
    text_num_attention_heads: int = 20
    text_num_kv_heads: int = 20

    @property
    def hidden_size(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @property
    def latent_channels(self) -> int:
        return self.in_channels // (self.patch_size * self.patch_size)

    def validate(self) -> None:
        if sum(self.axes_dims_rope) != self.attention_head_dim:
            raise ValueError("krea: axes_dims_rope must sum to attention_head_dim")
        if self.num_attention_heads % self.num_kv_heads or self.text_num_attention_heads % self.text_num_kv_heads:
            raise ValueError("krea: query heads must be a multiple of kv heads")
        if self.text_num_attention_heads * self.attention_head_dim != self.text_hidden_dim:
            raise ValueError("krea: text heads x head_dim must equal text_hidden_dim")

    @staticmethod
    def from_json(j: dict) -> "KreaConfig":
        d = {k: j[k] for k in KreaConfig.__dataclass_fields__ if k in j}
        if "axes_dims_rope" in d:
            d["axes_dims_rope"] = tuple(d["axes_dims_rope"])
        cfg = KreaConfig(**d)
        cfg.validate()
        return cfg


def _attn_names(p: str) -> list[str]:
    return [f"{p}.{n}" for n in ("to_q", "to_k", "to_v", "to_gate", "to_out.0")]


def random_krea_weights(cfg: KreaConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                        ) -> dict[str, torch.Tensor]:
    rn, lin = nd.randn_weights(seed, device)
    w: dict[str, torch.Tensor] = {}
    H, hd, Td = cfg.hidden_size, cfg.attention_head_dim, cfg.text_hidden_dim

    def block(p: str, width: int, heads: int, kv: int, ffn: int):
        for n, o, i in (("to_q", heads * hd, width), ("to_k", kv * hd, width), ("to_v", kv * hd, width),
                        ("to_gate", heads * hd, width), ("to_out.0", width, heads * hd)):
            lin(w, f"{p}.attn.{n}", o, i, std, bias=False, dtype=dtype)
        for n in ("norm_q", "norm_k"):
            w[f"{p}.attn.{n}.weight"] = (rn(hd) * 0.1).to(dtype)
        for n in ("norm1", "norm2"):
            w[f"{p}.{n}.weight"] = (rn(width) * 0.1).to(dtype)
        lin(w, f"{p}.ff.gate", ffn, width, std, bias=False, dtype=dtype)
        lin(w, f"{p}.ff.up", ffn, width, std, bias=False, dtype=dtype)
        lin(w, f"{p}.ff.down", width, ffn, std, bias=False, dtype=dtype)

    lin(w, "img_in", H, cfg.in_channels, std, dtype=dtype)
    lin(w, "time_embed.linear_1", H, cfg.timestep_embed_dim, std, dtype=dtype)
    lin(w, "time_embed.linear_2", H, H, std, dtype=dtype)
    lin(w, "time_mod_proj", 6 * H, H, std, dtype=dtype)
    w["txt_in.norm.weight"] = (rn(Td) * 0.1).to(dtype)
    lin(w, "txt_in.linear_1", H, Td, std, dtype=dtype)
    lin(w, "txt_in.linear_2", H, H, std, dtype=dtype)
    for i in range(cfg.num_layerwise_text_blocks):
        block(f"text_fusion.layerwise_blocks.{i}", Td, cfg.text_num_attention_heads, cfg.text_num_kv_heads,
              cfg.text_intermediate_size)
    w["text_fusion.projector.weight"] = (rn(1, cfg.num_text_layers) * 0.3).to(dtype)
    for i in range(cfg.num_refiner_text_blocks):
        block(f"text_fusion.refiner_blocks.{i}", Td, cfg.text_num_attention_heads, cfg.text_num_kv_heads,
              cfg.text_intermediate_size)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        block(p, H, cfg.num_attention_heads, cfg.num_kv_heads, cfg.intermediate_size)
        w[f"{p}.scale_shift_table"] = (rn(6, H) * 0.1).to(dtype)
    w["final_layer.norm.weight"] = (rn(H) * 0.1).to(dtype)
    w["final_layer.scale_shift_table"] = (rn(2, H) * 0.1).to(dtype)
    lin(w, "final_layer.linear", cfg.in_channels, H, std, dtype=dtype)
    return w


def krea_positions(cap_len: int, ht: int, wt: int, n_refs: int = 0) -> torch.Tensor:
    """[cap + (n_refs + 1) * ht * wt, 3] (frame, row, column): text at the origin, reference i at frame i + 1, the
    target image at frame 0 (candle-gen-krea/src/transformer/rope.rs:build_t2i / build_edit)."""
    rows = torch.arange(ht, dtype=torch.float32)[:, None].expand(ht, wt).reshape(-1)
    cols = torch.arange(wt, dtype=torch.float32)[None, :].expand(ht, wt).reshape(-1)
    parts = [torch.zeros(cap_len, 3)]
    for i in range(n_refs):
        parts.append(torch.stack((torch.full_like(rows, float(i + 1)), rows, cols), dim=1))
    parts.append(torch.stack((torch.zeros_like(rows), rows, cols), dim=1))
    return torch.cat(parts, dim=0)


class KreaDiT:
    """fp32 oracle on CPU, bf16 on the sm_100a kernels on a CUDA device (see the module docstring)."""

    FUSED = ("to_qkvg", "ff.gate_up")

    def __init__(self, cfg: KreaConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        cfg.validate()
        self.cfg = cfg
        self.bag = nd.WeightBag(weights, dtype, device)
        self.dtype, self.device = self.bag.dtype, self.bag.device
        w = self.bag.w
        # "RMS scale": weight = scale + 1 (stored as the offset of the norm kernel)
        self._rope_cache: dict[tuple[int, int, int, int], tuple[torch.Tensor, torch.Tensor]] = {}
        self.nvfp4 = None            # name -> packed projection after quantize_nvfp4()
        self.lora = None             # training: {module name: (A [r, in], B [out, r], scale)}, added to the projection's output
        if self.device.type == "cuda":
            # one GEMM for q / k / v / gate and one for the SwiGLU gate / up pair of every block
            for p in self._block_prefixes():
                a = p + ".attn."
                w[a + "to_qkvg.weight"] = torch.cat([w.pop(a + n + ".weight") for n in ("to_q", "to_k", "to_v", "to_gate")])
                w[p + ".ff.gate_up.weight"] = torch.cat([w.pop(p + ".ff.gate.weight"), w.pop(p + ".ff.up.weight")])

    def _block_prefixes(self) -> list[str]:
        c = self.cfg
        return ([f"text_fusion.layerwise_blocks.{i}" for i in range(c.num_layerwise_text_blocks)] +
                [f"text_fusion.refiner_blocks.{i}" for i in range(c.num_refiner_text_blocks)] +
                [f"transformer_blocks.{i}" for i in range(c.num_layers)])

    def weight_bytes(self) -> int:
        n = self.bag.nbytes()
        if self.nvfp4:
            n += sum(q.nvfp4_footprint_bytes() for q in self.nvfp4.values())
        return n

    # ---- pieces ------------------------------------------------------------------------------------------------------
    def _proj(self, x: torch.Tensor, name: str) -> torch.Tensor:
        if self.nvfp4 is not None and name in self.nvfp4:
            return self.nvfp4[name](x)
        y = self.bag.lin(x, name)
        if self.lora is not None and name in self.lora:
            y = y + nd.adapter_residual(self.lora[name], x)
        return y

    def _rms(self, x: torch.Tensor, key: str) -> torch.Tensor:
        return nd.rms_norm(x, self.bag[key], self.cfg.norm_eps, offset=1.0)

    def _attention(self, x: torch.Tensor, p: str, heads: int, kv: int, rope) -> torch.Tensor:
        B, S, _ = x.shape
        hd = self.cfg.attention_head_dim
        a = p + ".attn."
        if (a + "to_qkvg.weight") in self.bag or (self.nvfp4 is not None and (a + "to_qkvg") in self.nvfp4):
            y = self._proj(x, a + "to_qkvg")
            q, k, v, gate = y.split((heads * hd, kv * hd, kv * hd, heads * hd), dim=-1)
        else:
            q, k, v, gate = (self._proj(x, a + n) for n in ("to_q", "to_k", "to_v", "to_gate"))
        q = self._rms(q.reshape(B, S, heads, hd), a + "norm_q.weight")
        k = self._rms(k.reshape(B, S, kv, hd), a + "norm_k.weight")
        v = v.reshape(B, S, kv, hd)
        if rope is not None:
            q, k = nd.rope_interleaved(q, *rope), nd.rope_interleaved(k, *rope)
        o = nd.attention(q, k, v, scale=hd ** -0.5)
        return self._proj(o * torch.sigmoid(gate.float()).to(o.dtype), a + "to_out.0")

    def _swiglu(self, x: torch.Tensor, p: str) -> torch.Tensor:
        f = p + ".ff."
        if (f + "gate_up.weight") in self.bag or (self.nvfp4 is not None and (f + "gate_up") in self.nvfp4):
            g, u = self._proj(x, f + "gate_up").chunk(2, dim=-1)
        else:
            g, u = self._proj(x, f + "gate"), self._proj(x, f + "up")
        return self._proj((F.silu(g.float()) * u.float()).to(x.dtype), f + "down")

    def _fusion_block(self, x: torch.Tensor, p: str) -> torch.Tensor:
        c = self.cfg
        x = x + self._attention(self._rms(x, p + ".norm1.weight"), p, c.text_num_attention_heads, c.text_num_kv_heads, None)
        return x + self._swiglu(self._rms(x, p + ".norm2.weight"), p)

    def text_fusion(self, context: torch.Tensor) -> torch.Tensor:
        """[B, L, num_text_layers, text_hidden] -> [B, L, hidden]. Independent of the timestep: a pipeline calls it
        once per prompt."""
        c = self.cfg
        B, L, NL, D = context.shape
        h = context.to(self.device, self.dtype).reshape(B * L, NL, D)
        for i in range(c.num_layerwise_text_blocks):
            h = self._fusion_block(h, f"text_fusion.layerwise_blocks.{i}")
        pw = self.bag["text_fusion.projector.weight"].float().view(NL)            # Linear(12 -> 1), no bias
        h = (h.float() * pw[None, :, None]).sum(1).to(self.dtype).reshape(B, L, D)
        for i in range(c.num_refiner_text_blocks):
            h = self._fusion_block(h, f"text_fusion.refiner_blocks.{i}")
        h = self._rms(h, "txt_in.norm.weight")
        return self.bag.lin(self.bag.lin(h, "txt_in.linear_1", act="gelu"), "txt_in.linear_2")

    def rope(self, cap_len: int, ht: int, wt: int, n_refs: int = 0):
        key = (cap_len, ht, wt, n_refs)
        if key not in self._rope_cache:
            if len(self._rope_cache) >= 4:
                self._rope_cache.pop(next(iter(self._rope_cache)))
            cos, sin = nd.axis_rope_tables(krea_positions(cap_len, ht, wt, n_refs), self.cfg.axes_dims_rope,
                                           self.cfg.rope_theta)
            self._rope_cache[key] = (cos.to(self.device), sin.to(self.device))
        return self._rope_cache[key]

    # ---- forward -------------------------------------------------------------------------------------------------------
    def forward_grad(self, latent: torch.Tensor, timestep: torch.Tensor, context: torch.Tensor,
                     refs: list[torch.Tensor] | None = None, fused_context: torch.Tensor | None = None) -> torch.Tensor:
        """latent [B, C, H, W]; timestep [B] (sigma; scaled x 1000 inside); context [B, L, 12, text_hidden] (or
        `fused_context` = text_fusion(context), [B, L, hidden]); refs: reference latents of an edit, each [B, C, H, W]
        -> flow velocity [B, C, H, W]."""
        c = self.cfg
        p = c.patch_size
        B, _, Hh, Ww = latent.shape
        ht, wt = Hh // p, Ww // p
        dev, dt = self.device, self.dtype
        img = self.bag.lin(nd.patchify(latent.to(dev, dt), p), "img_in")
        refs = refs or []
        for i, r in enumerate(refs):
            if r.shape[-2:] != latent.shape[-2:]:
                raise ValueError(f"krea edit: reference {i} is {tuple(r.shape[-2:])} but the target latent is "
                                 f"{tuple(latent.shape[-2:])}; references must be encoded at the target resolution")
        ref_tok = [self.bag.lin(nd.patchify(r.to(dev, dt), p), "img_in") for r in refs]
        t_sin = nd.sinusoidal_embedding(timestep.to(dev), c.timestep_embed_dim, scale=1000.0).to(dt)[:, None, :]
        t = self.bag.lin(self.bag.lin(t_sin, "time_embed.linear_1", act="gelu"), "time_embed.linear_2")     # [B, 1, H]
        tvec = self.bag.lin(F.gelu(t.float()).to(dt), "time_mod_proj")                                      # [B, 1, 6H]
        ctx = fused_context.to(dev, dt) if fused_context is not None else self.text_fusion(context)
        cap = ctx.shape[1]
        x = torch.cat([ctx, *ref_tok, img], dim=1)
        rope = self.rope(cap, ht, wt, len(refs))
        H = c.hidden_size
        for i in range(c.num_layers):
            bp = f"transformer_blocks.{i}"
            m = (tvec.float() + self.bag[bp + ".scale_shift_table"].float().reshape(1, 1, 6 * H)).to(dt)
            prs, prh, prg, pos, poh, pog = m.chunk(6, dim=-1)
            h = self._rms(x, bp + ".norm1.weight") * (1 + prs) + prh
            x = x + self._attention(h, bp, c.num_attention_heads, c.num_kv_heads, rope) * prg
            h = self._rms(x, bp + ".norm2.weight") * (1 + pos) + poh
            x = x + self._swiglu(h, bp) * pog
        fm = (t.float() + self.bag["final_layer.scale_shift_table"].float().reshape(1, 2, H)).to(dt)
        scale, shift = fm[:, 0:1], fm[:, 1:2]
        out = self.bag.lin(self._rms(x, "final_layer.norm.weight") * (1 + scale) + shift, "final_layer.linear")
        n_img = ht * wt
        start = cap + len(refs) * n_img
        return nd.unpatchify(out[:, start:start + n_img], ht, wt, p, c.latent_channels)

    @torch.no_grad()
    def forward(self, latent, timestep, context, refs=None, fused_context=None):
        return self.forward_grad(latent, timestep, context, refs, fused_context)

    # ---- NVFP4 -----------------------------------------------------------------------------------------------------------
    def quantize_nvfp4(self, act: str = "w4a16", skip_first_last: int = 0) -> dict:
        """Repacks the attention and SwiGLU projections of the single-stream blocks to NVFP4 (E2M1 codes in 16-element
        blocks, E4M3 block scales, one fp32 tensor scale; the role of candle-gen-krea/src/nvfp4_dit.rs). `act`:
        "w4a16" keeps bf16 activations, "w4a4" also rounds the activations to the NVFP4 grid per 16-element block.
        The first / last `skip_first_last` blocks stay dense (the reference's mixed plan). Device only.
        Returns a report {layers, bytes_before, bytes_after}."""
        from ..ops.nvfp4 import ActPrecision, Nvfp4Linear, quantize_on_device

        if self.device.type != "cuda":
            raise RuntimeError("quantize_nvfp4 needs the CUDA backend")
        before = self.weight_bytes()
        self.nvfp4 = {}
        n = self.cfg.num_layers
        for i in range(n):
            if i < skip_first_last or i >= n - skip_first_last:
                continue
            bp = f"transformer_blocks.{i}"
            for name in (bp + ".attn.to_qkvg", bp + ".attn.to_out.0", bp + ".ff.gate_up", bp + ".ff.down"):
                wt = self.bag.w.pop(name + ".weight")
                self.nvfp4[name] = Nvfp4Linear(quantize_on_device(wt), None,
                                               ActPrecision.W4A4 if act == "w4a4" else ActPrecision.W4A16)
                del wt
        torch.cuda.empty_cache()
        return {"layers": len(self.nvfp4), "bytes_before": before, "bytes_after": self.weight_bytes(), "act": act}
