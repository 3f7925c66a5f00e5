"""Qwen-Image MMDiT (parity: candle-gen-qwen-image/src/transformer.rs, rope.rs, config.rs; checkpoint keys are the
diffusers `QwenImageTransformer2DModel` names).

Sixty dual-stream blocks and nothing else: each block is the FLUX double block (per-stream adaLN-Zero modulation,
q/k/v with per-head RMSNorm, joint attention over [text, image] with interleaved three-axis RoPE, GELU-tanh MLPs).
The conditioning vector is the timestep embedding alone; the text features pass an RMSNorm before `txt_in`; the output
layer's modulation is stored (scale, shift). So the checkpoint is converted to the fused FLUX layout and runs on the
FLUX implementations (oracle and sm_100a, sequence-parallel included) with three overrides: the conditioning vector,
the position ids (image rows / columns are centred on zero, text positions start past the image's half-extent on all
three axes) and the text pre-norm, which is hoisted out of the step loop."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT, timestep_embedding


@dataclass
class QwenImageConfig:
    in_channels: int = 64
    num_layers: int = 60
    attention_head_dim: int = 128
    num_attention_heads: int = 24
    joint_attention_dim: int = 3584
    axes_dims_rope: tuple[int, int, int] = (16, 56, 56)
    rope_theta: float = 10000.0

    @property
    def inner_dim(self) -> int:
        return self.attention_head_dim * self.num_attention_heads

    def flux_config(self) -> FluxConfig:
        return FluxConfig(in_channels=self.in_channels, vec_in_dim=8, context_in_dim=self.joint_attention_dim,
                          hidden_size=self.inner_dim, num_heads=self.num_attention_heads, depth=self.num_layers,
                          depth_single=0, axes_dim=tuple(self.axes_dims_rope), theta=self.rope_theta,
                          guidance_embed=False)

    @staticmethod
    def from_json(j: dict) -> "QwenImageConfig":
        d = {k: j[k] for k in QwenImageConfig.__dataclass_fields__ if k in j}
        if "axes_dims_rope" in d:
            d["axes_dims_rope"] = tuple(d["axes_dims_rope"])
        return QwenImageConfig(**d)


def convert_qwen_image_weights(sd: dict[str, torch.Tensor], cfg: QwenImageConfig) -> dict[str, torch.Tensor]:
    """diffusers names -> the fused FLUX layout (+ `txt_norm.weight` kept as it is)."""
    out: dict[str, torch.Tensor] = {"txt_norm.weight": sd["txt_norm.weight"]}

    def take(dst: str, src: str) -> None:
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = sd[f"{src}.{leaf}"]

    def fuse(dst: str, srcs: list[str]) -> None:
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = torch.cat([sd[f"{s}.{leaf}"] for s in srcs], dim=0)

    take("img_in", "img_in")
    take("txt_in", "txt_in")
    take("time_in.in_layer", "time_text_embed.timestep_embedder.linear_1")
    take("time_in.out_layer", "time_text_embed.timestep_embedder.linear_2")
    take("final_layer.linear", "proj_out")
    H = cfg.inner_dim
    for leaf in ("weight", "bias"):                        # stored (scale, shift); the FLUX layout reads (shift, scale)
        t = sd[f"norm_out.linear.{leaf}"]
        out[f"final_layer.adaLN_modulation.1.{leaf}"] = torch.cat([t[H:], t[:H]], 0)
    for i in range(cfg.num_layers):
        s, d = f"transformer_blocks.{i}", f"double_blocks.{i}"
        take(f"{d}.img_mod.lin", f"{s}.img_mod.1")
        take(f"{d}.txt_mod.lin", f"{s}.txt_mod.1")
        fuse(f"{d}.img_attn.qkv", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v"])
        fuse(f"{d}.txt_attn.qkv", [f"{s}.attn.add_q_proj", f"{s}.attn.add_k_proj", f"{s}.attn.add_v_proj"])
        take(f"{d}.img_attn.proj", f"{s}.attn.to_out.0")
        take(f"{d}.txt_attn.proj", f"{s}.attn.to_add_out")
        out[f"{d}.img_attn.norm.query_norm.scale"] = sd[f"{s}.attn.norm_q.weight"]
        out[f"{d}.img_attn.norm.key_norm.scale"] = sd[f"{s}.attn.norm_k.weight"]
        out[f"{d}.txt_attn.norm.query_norm.scale"] = sd[f"{s}.attn.norm_added_q.weight"]
        out[f"{d}.txt_attn.norm.key_norm.scale"] = sd[f"{s}.attn.norm_added_k.weight"]
        take(f"{d}.img_mlp.0", f"{s}.img_mlp.net.0.proj")
        take(f"{d}.img_mlp.2", f"{s}.img_mlp.net.2")
        take(f"{d}.txt_mlp.0", f"{s}.txt_mlp.net.0.proj")
        take(f"{d}.txt_mlp.2", f"{s}.txt_mlp.net.2")
    return out


def random_qwen_image_weights(cfg: QwenImageConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                              ) -> dict[str, torch.Tensor]:
    """A random checkpoint in the diffusers layout."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device)      # noqa: E731
    H, M = cfg.inner_dim, 4 * cfg.inner_dim
    w: dict[str, torch.Tensor] = {}

    def lin(name, o, i):
        w[name + ".weight"], w[name + ".bias"] = (rn(o, i) * std).to(dtype), (rn(o) * std).to(dtype)

    lin("img_in", H, cfg.in_channels)
    lin("txt_in", H, cfg.joint_attention_dim)
    w["txt_norm.weight"] = (1.0 + rn(cfg.joint_attention_dim) * 0.1).to(dtype)
    lin("time_text_embed.timestep_embedder.linear_1", H, 256)
    lin("time_text_embed.timestep_embedder.linear_2", H, H)
    lin("norm_out.linear", 2 * H, H)
    lin("proj_out", cfg.in_channels, H)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        lin(f"{p}.img_mod.1", 6 * H, H)
        lin(f"{p}.txt_mod.1", 6 * H, H)
        for n in ("to_q", "to_k", "to_v", "to_out.0", "add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"):
            lin(f"{p}.attn.{n}", H, H)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            w[f"{p}.attn.{n}.weight"] = (1.0 + rn(cfg.attention_head_dim) * 0.1).to(dtype)
        for s in ("img_mlp", "txt_mlp"):
            lin(f"{p}.{s}.net.0.proj", M, H)
            lin(f"{p}.{s}.net.2", H, M)
    return w


def position_ids(h_tokens: int, w_tokens: int, txt_len: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """(text ids [L, 3], image ids [h*w, 3]). Image token (r, c) sits at (0, r - (h - h//2), c - (w - w//2)); text
    token t sits at max(h//2, w//2) + t on all three axes."""
    img = torch.zeros(h_tokens, w_tokens, 3, device=device)
    img[..., 1] = (torch.arange(h_tokens, device=device) - (h_tokens - h_tokens // 2))[:, None]
    img[..., 2] = (torch.arange(w_tokens, device=device) - (w_tokens - w_tokens // 2))[None, :]
    base = max(h_tokens // 2, w_tokens // 2)
    txt = (base + torch.arange(txt_len, device=device, dtype=torch.float32))[:, None].expand(txt_len, 3).contiguous()
    return txt, img.reshape(-1, 3)


def _text_prenorm(txt: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    xf = txt.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * weight.float()).to(weight.dtype)


class OracleQwenImageDiT(OracleFluxDiT):
    def __init__(self, cfg: QwenImageConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.qcfg = cfg
        super().__init__(cfg.flux_config(), convert_qwen_image_weights(weights, cfg), dtype, device)

    def prepare_text(self, txt: torch.Tensor) -> torch.Tensor:
        """Encoder features -> the `txt` argument of forward (the RMSNorm in front of `txt_in`)."""
        return _text_prenorm(txt.to(self.w["txt_norm.weight"].device), self.w["txt_norm.weight"])

    def _modulations(self, timesteps, y, guidance, dtype):
        cfg = self.cfg
        sv = F.silu(self._mlp_embed(timestep_embedding(timesteps).to(dtype), "time_in"))
        names = [f"double_blocks.{i}.{s}_mod.lin" for i in range(cfg.depth) for s in ("img", "txt")]
        return {n: self._lin(sv, n) for n in names + ["final_layer.adaLN_modulation.1"]}


class QwenImageDiTGpu(FluxDiTGpu):
    def __init__(self, cfg: QwenImageConfig, comm=None, device=None):
        self.qcfg = cfg
        super().__init__(cfg.flux_config(), comm, device)

    def load_state_dict(self, weights: dict[str, torch.Tensor]) -> "QwenImageDiTGpu":
        return super().load_state_dict(convert_qwen_image_weights(weights, self.qcfg))

    def init_random(self, seed: int = 0, std: float = 0.02) -> "QwenImageDiTGpu":
        return self.load_state_dict(random_qwen_image_weights(self.qcfg, seed, std, torch.bfloat16, self.device))

    def prepare_text(self, txt: torch.Tensor) -> torch.Tensor:
        from .. import ops

        t = txt.to(self.device, torch.bfloat16).contiguous()
        return ops.rmsnorm(t.view(-1, t.shape[-1]), self.w["txt_norm.weight"], 1e-6).view(t.shape)

    def conditioning_vector(self, timesteps, y, guidance) -> torch.Tensor:
        vec = self._embed(timestep_embedding(timesteps.to(self.device)).bfloat16(), "time_in")
        return F.silu(vec.float()).bfloat16().contiguous()
