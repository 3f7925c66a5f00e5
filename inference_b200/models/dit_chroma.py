"""Chroma DiT: the FLUX.1 transformer skeleton whose per-block modulation linears are replaced by one small
"distilled guidance" network (the Approximator), conditioned on T5 only (candle-gen-chroma/src/transformer.rs).

The Approximator turns (timestep embedding, zero-guidance embedding, modulation-index embedding) into a table of
344 hidden-sized vectors per sample: 3 per single block (shift, scale, gate), 6 per double block for the image
stream, 6 for the text stream, 2 for the final layer. Everything downstream is the FLUX block math, so both the
fp32 oracle and the sm_100a model subclass the FLUX ones and only swap where the modulations come from: a Chroma
checkpoint (diffusers key names, separate q / k / v projections) is converted once at load into the fused layout
those classes use."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .dit_flux import FluxConfig, FluxDiTGpu, OracleFluxDiT

APPROX_RMS_EPS = 1.1920929e-07


@dataclass
class ChromaConfig:
    in_channels: int = 64
    num_layers: int = 19
    num_single_layers: int = 38
    attention_head_dim: int = 128
    num_attention_heads: int = 24
    joint_attention_dim: int = 4096
    axes_dims_rope: tuple[int, int, int] = (16, 56, 56)
    approximator_num_channels: int = 64
    approximator_hidden_dim: int = 5120
    approximator_layers: int = 5

    @property
    def inner_dim(self) -> int:
        return self.attention_head_dim * self.num_attention_heads

    @property
    def mod_index_len(self) -> int:
        return 3 * self.num_single_layers + 12 * self.num_layers + 2

    def flux_config(self) -> FluxConfig:
        return FluxConfig(in_channels=self.in_channels, vec_in_dim=8, context_in_dim=self.joint_attention_dim,
                          hidden_size=self.inner_dim, num_heads=self.num_attention_heads, depth=self.num_layers,
                          depth_single=self.num_single_layers, axes_dim=tuple(self.axes_dims_rope), guidance_embed=False)

    @staticmethod
    def from_json(j: dict) -> "ChromaConfig":
        keys = ChromaConfig.__dataclass_fields__
        d = {k: j[k] for k in keys if k in j}
        if "axes_dims_rope" in d:
            d["axes_dims_rope"] = tuple(d["axes_dims_rope"])
        return ChromaConfig(**d)


# ---- checkpoint conversion (diffusers names -> the fused FLUX layout) --------------------------------------------------------
def convert_chroma_weights(sd: dict[str, torch.Tensor], cfg: ChromaConfig) -> dict[str, torch.Tensor]:
    out: dict[str, torch.Tensor] = {}

    def take(dst: str, src: str) -> None:
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = sd[f"{src}.{leaf}"]

    def fuse(dst: str, srcs: list[str]) -> None:
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = torch.cat([sd[f"{s}.{leaf}"] for s in srcs], dim=0)

    take("img_in", "x_embedder")
    take("txt_in", "context_embedder")
    take("final_layer.linear", "proj_out")
    for i in range(cfg.num_layers):
        s, d = f"transformer_blocks.{i}", f"double_blocks.{i}"
        fuse(f"{d}.img_attn.qkv", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v"])
        fuse(f"{d}.txt_attn.qkv", [f"{s}.attn.add_q_proj", f"{s}.attn.add_k_proj", f"{s}.attn.add_v_proj"])
        take(f"{d}.img_attn.proj", f"{s}.attn.to_out.0")
        take(f"{d}.txt_attn.proj", f"{s}.attn.to_add_out")
        out[f"{d}.img_attn.norm.query_norm.scale"] = sd[f"{s}.attn.norm_q.weight"]
        out[f"{d}.img_attn.norm.key_norm.scale"] = sd[f"{s}.attn.norm_k.weight"]
        out[f"{d}.txt_attn.norm.query_norm.scale"] = sd[f"{s}.attn.norm_added_q.weight"]
        out[f"{d}.txt_attn.norm.key_norm.scale"] = sd[f"{s}.attn.norm_added_k.weight"]
        take(f"{d}.img_mlp.0", f"{s}.ff.net.0.proj")
        take(f"{d}.img_mlp.2", f"{s}.ff.net.2")
        take(f"{d}.txt_mlp.0", f"{s}.ff_context.net.0.proj")
        take(f"{d}.txt_mlp.2", f"{s}.ff_context.net.2")
    for i in range(cfg.num_single_layers):
        s, d = f"single_transformer_blocks.{i}", f"single_blocks.{i}"
        fuse(f"{d}.linear1", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v", f"{s}.proj_mlp"])
        take(f"{d}.linear2", f"{s}.proj_out")
        out[f"{d}.norm.query_norm.scale"] = sd[f"{s}.attn.norm_q.weight"]
        out[f"{d}.norm.key_norm.scale"] = sd[f"{s}.attn.norm_k.weight"]
    for k, v in sd.items():
        if k.startswith("distilled_guidance_layer."):
            out[k] = v
    return out


def random_chroma_weights(cfg: ChromaConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                          ) -> dict[str, torch.Tensor]:
    """A random checkpoint in the diffusers layout (tests, synthetic snapshots)."""
    g = torch.Generator(device=device).manual_seed(seed)
    rn = lambda *shape: torch.randn(*shape, generator=g, device=device)      # noqa: E731
    H, M = cfg.inner_dim, 4 * cfg.inner_dim
    w: dict[str, torch.Tensor] = {}

    def lin(name, o, i):
        w[name + ".weight"], w[name + ".bias"] = (rn(o, i) * std).to(dtype), (rn(o) * std).to(dtype)

    lin("x_embedder", H, cfg.in_channels)
    lin("context_embedder", H, cfg.joint_attention_dim)
    lin("proj_out", cfg.in_channels, H)
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}"
        for n in ("to_q", "to_k", "to_v", "to_out.0", "add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"):
            lin(f"{p}.attn.{n}", H, H)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            w[f"{p}.attn.{n}.weight"] = (1.0 + rn(cfg.attention_head_dim) * 0.1).to(dtype)
        for ff in ("ff", "ff_context"):
            lin(f"{p}.{ff}.net.0.proj", M, H)
            lin(f"{p}.{ff}.net.2", H, M)
    for i in range(cfg.num_single_layers):
        p = f"single_transformer_blocks.{i}"
        for n in ("to_q", "to_k", "to_v"):
            lin(f"{p}.attn.{n}", H, H)
        for n in ("norm_q", "norm_k"):
            w[f"{p}.attn.{n}.weight"] = (1.0 + rn(cfg.attention_head_dim) * 0.1).to(dtype)
        lin(f"{p}.proj_mlp", M, H)
        lin(f"{p}.proj_out", H, H + M)
    a, hid = "distilled_guidance_layer", cfg.approximator_hidden_dim
    lin(f"{a}.in_proj", hid, cfg.approximator_num_channels)
    for i in range(cfg.approximator_layers):
        lin(f"{a}.layers.{i}.linear_1", hid, hid)
        lin(f"{a}.layers.{i}.linear_2", hid, hid)
        w[f"{a}.norms.{i}.weight"] = (1.0 + rn(hid) * 0.1).to(dtype)
    lin(f"{a}.out_proj", H, hid)
    return w


# ---- the Approximator ----------------------------------------------------------------------------------------------------
def _cos_sin_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """[N] -> [N, dim]: cos block then sin block, frequencies exp(-ln(10000) * i / (dim / 2))."""
    half = dim // 2
    freqs = torch.exp(torch.arange(half, dtype=torch.float32, device=t.device) * (-math.log(10000.0) / half))
    e = t.float().reshape(-1, 1) * freqs[None, :]
    return torch.cat([e.cos(), e.sin()], dim=-1)


def approximator_input(timesteps: torch.Tensor, cfg: ChromaConfig) -> torch.Tensor:
    """[B] flow times in [0, 1] -> [B, N, 4 nc]: (time, zero guidance) embeddings repeated over the N modulation
    slots, next to each slot's index embedding."""
    nc = cfg.approximator_num_channels // 4
    n = cfg.mod_index_len
    dev = timesteps.device
    t = timesteps.float().flatten() * 1000.0
    tg = torch.cat([_cos_sin_embedding(t, nc), _cos_sin_embedding(torch.zeros_like(t), nc)], dim=-1)
    idx = _cos_sin_embedding(torch.arange(n, dtype=torch.float32, device=dev) * 1000.0, 2 * nc)
    b = t.numel()
    return torch.cat([tg[:, None, :].expand(b, n, 2 * nc), idx[None].expand(b, n, 2 * nc)], dim=-1)


def approximator_forward(lin, norm_w, x: torch.Tensor, layers: int) -> torch.Tensor:
    """lin(name, x) applies `distilled_guidance_layer.<name>`; norm_w(i) is the i-th RMSNorm weight."""
    x = lin("in_proj", x)
    for i in range(layers):
        xf = x.float()
        n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + APPROX_RMS_EPS)).to(x.dtype) * norm_w(i)
        x = x + lin(f"layers.{i}.linear_2", F.silu(lin(f"layers.{i}.linear_1", n).float()).to(x.dtype))
    return lin("out_proj", x)


def table_to_modulations(table: torch.Tensor, cfg: ChromaConfig) -> dict[str, torch.Tensor]:
    """[B, N, H] -> the FLUX modulation dictionary: consecutive rows concatenated per block."""
    b = table.shape[0]
    ns, nd = cfg.num_single_layers, cfg.num_layers
    img0, txt0 = 3 * ns, 3 * ns + 6 * nd
    out = {}
    for i in range(nd):
        out[f"double_blocks.{i}.img_mod.lin"] = table[:, img0 + 6 * i: img0 + 6 * i + 6].reshape(b, -1)
        out[f"double_blocks.{i}.txt_mod.lin"] = table[:, txt0 + 6 * i: txt0 + 6 * i + 6].reshape(b, -1)
    for i in range(ns):
        out[f"single_blocks.{i}.modulation.lin"] = table[:, 3 * i: 3 * i + 3].reshape(b, -1)
    out["final_layer.adaLN_modulation.1"] = table[:, -2:].reshape(b, -1)
    return out


# ---- models --------------------------------------------------------------------------------------------------------------
class OracleChromaDiT(OracleFluxDiT):
    def __init__(self, cfg: ChromaConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.ccfg = cfg
        super().__init__(cfg.flux_config(), convert_chroma_weights(weights, cfg), dtype, device)

    def _modulations(self, timesteps, y, guidance, dtype):
        a = "distilled_guidance_layer."
        x = approximator_input(timesteps.to(self.w["img_in.weight"].device), self.ccfg).to(dtype)
        table = approximator_forward(lambda n, t: self._lin(t, a + n), lambda i: self.w[f"{a}norms.{i}.weight"], x,
                                     self.ccfg.approximator_layers)
        return table_to_modulations(table, self.ccfg)


class ChromaDiTGpu(FluxDiTGpu):
    """The sm_100a FLUX model with the Approximator as its modulation source (all of its projections on the
    tcgen05 GEMM: the table is 344 rows, so each of its eleven linears is one [344, 5120]-sized GEMM per step)."""

    def __init__(self, cfg: ChromaConfig, comm=None, device=None):
        self.ccfg = cfg
        super().__init__(cfg.flux_config(), comm, device)

    def load_state_dict(self, weights: dict[str, torch.Tensor]) -> "ChromaDiTGpu":
        return super().load_state_dict(convert_chroma_weights(weights, self.ccfg))

    def init_random(self, seed: int = 0, std: float = 0.02) -> "ChromaDiTGpu":
        return self.load_state_dict(random_chroma_weights(self.ccfg, seed, std, torch.bfloat16, self.device))

    def _build_modulation_table(self) -> None:       # no per-block modulation linears in this family
        return None

    def conditioning_vector(self, timesteps, y, guidance) -> torch.Tensor:
        return approximator_input(timesteps.to(self.device), self.ccfg).to(torch.bfloat16)

    def _all_modulations(self, sv: torch.Tensor) -> dict[str, torch.Tensor]:
        a = "distilled_guidance_layer."
        b, n, c = sv.shape

        def lin(name, t):
            return self._lin(t.reshape(-1, t.shape[-1]).contiguous(), a + name).view(b, n, -1)
        table = approximator_forward(lin, lambda i: self.w[f"{a}norms.{i}.weight"], sv, self.ccfg.approximator_layers)
        return {k: v.contiguous() for k, v in table_to_modulations(table, self.ccfg).items()}
