"""Z-Image single-stream DiT (parity: candle-gen-z-image/src/dit.rs; checkpoint keys are the diffusers
`ZImageTransformer2DModel` names).

Structure: a 256-wide timestep embedding drives every modulation; image patches go through `n_refiner_layers`
modulated blocks, caption features (RMSNorm + linear) through as many unmodulated blocks, then [image, caption] runs
through `n_layers` modulated blocks and the final layer projects the image rows back to patches. Every block is
sandwich-normed: x += tanh(gate) * RMSNorm2(f(RMSNorm1(x) * (1 + scale))) for f = attention (per-head q/k RMSNorm,
three-axis interleaved RoPE, full multi-head attention) and f = SwiGLU.

`OracleZImageDiT` is the fp32 PyTorch statement of that computation. `ZImageDiTGpu` runs it on the sm_100a kernels:
q/k/v as one GEMM, w1/w3 as one gated-pair GEMM, the (1 + scale) factors folded into per-step RMSNorm weights, all
modulation linears as one GEMM per step, and the caption branch (which does not depend on the timestep) computed once
per prompt instead of once per step."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .nn_dual import adapter_residual

from .dit_flux import rope_table

ADALN_DIM = 256
SEQ_MULTIPLE = 32          # caption lengths are counted in multiples of this when image positions are assigned


@dataclass
class ZImageConfig:
    dim: int = 3840
    n_layers: int = 30
    n_refiner_layers: int = 2
    n_heads: int = 30
    in_channels: int = 16
    patch_size: int = 2
    cap_feat_dim: int = 2560
    norm_eps: float = 1e-5
    rope_theta: float = 256.0
    t_scale: float = 1000.0
    axes_dims: tuple[int, int, int] = (32, 48, 48)

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def ffn_dim(self) -> int:
        return int(self.dim / 3 * 8)

    @property
    def adaln_dim(self) -> int:
        return min(self.dim, ADALN_DIM)

    @property
    def patch_dim(self) -> int:
        return self.patch_size * self.patch_size * self.in_channels

    @staticmethod
    def from_json(j: dict) -> "ZImageConfig":
        d = {k: j[k] for k in ZImageConfig.__dataclass_fields__ if k in j}
        if "axes_dims" in d:
            d["axes_dims"] = tuple(d["axes_dims"])
        if "all_patch_size" in j:
            d["patch_size"] = int(j["all_patch_size"][0])
        return ZImageConfig(**d)


def block_names(cfg: ZImageConfig) -> list[tuple[str, bool]]:
    """(key prefix, modulated) for every block in execution order of their families."""
    out = [(f"noise_refiner.{i}", True) for i in range(cfg.n_refiner_layers)]
    out += [(f"context_refiner.{i}", False) for i in range(cfg.n_refiner_layers)]
    return out + [(f"layers.{i}", True) for i in range(cfg.n_layers)]


def random_zimage_weights(cfg: ZImageConfig, seed: int = 0, std: float = 0.05, dtype=torch.float32, device="cpu"
                          ) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    w: dict[str, torch.Tensor] = {}
    D, Fd, A = cfg.dim, cfg.ffn_dim, cfg.adaln_dim

    def lin(name, o, i, bias=True):
        w[name + ".weight"] = (torch.randn(o, i, generator=g, device=device) * std).to(dtype)
        if bias:
            w[name + ".bias"] = (torch.randn(o, generator=g, device=device) * std).to(dtype)

    def norm(name, n):
        w[name + ".weight"] = (1.0 + torch.randn(n, generator=g, device=device) * 0.1).to(dtype)

    lin("t_embedder.mlp.0", 1024, 256)
    lin("t_embedder.mlp.2", A, 1024)
    norm("cap_embedder.0", cfg.cap_feat_dim)
    lin("cap_embedder.1", D, cfg.cap_feat_dim)
    lin("all_x_embedder.2-1", D, cfg.patch_dim)
    lin("all_final_layer.2-1.linear", cfg.patch_dim, D)
    lin("all_final_layer.2-1.adaLN_modulation.1", D, A)
    w["x_pad_token"], w["cap_pad_token"] = torch.zeros(1, D, dtype=dtype), torch.zeros(1, D, dtype=dtype)
    for p, modulated in block_names(cfg):
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            lin(f"{p}.attention.{n}", D, D, bias=False)
        norm(f"{p}.attention.norm_q", cfg.head_dim)
        norm(f"{p}.attention.norm_k", cfg.head_dim)
        lin(f"{p}.feed_forward.w1", Fd, D, bias=False)
        lin(f"{p}.feed_forward.w3", Fd, D, bias=False)
        lin(f"{p}.feed_forward.w2", D, Fd, bias=False)
        for n in ("attention_norm1", "attention_norm2", "ffn_norm1", "ffn_norm2"):
            norm(f"{p}.{n}", D)
        if modulated:
            lin(f"{p}.adaLN_modulation.0", 4 * D, A)
    return w


# ---- token layout ------------------------------------------------------------------------------------------------------------
def patchify(z: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), p*p*C]; inside a patch the channel index runs fastest."""
    B, C, H, W = z.shape
    return z.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(B, (H // p) * (W // p), p * p * C)


def unpatchify(x: torch.Tensor, h: int, w: int, p: int = 2) -> torch.Tensor:
    """Inverse of patchify for a latent of h x w."""
    B, _, PD = x.shape
    C = PD // (p * p)
    return x.reshape(B, h // p, w // p, p, p, C).permute(0, 5, 1, 3, 2, 4).reshape(B, C, h, w)


def position_ids(h_tokens: int, w_tokens: int, cap_len: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """(image ids [h*w, 3], caption ids [cap_len, 3]). Caption token i sits at (1 + i, 0, 0); the image plane sits one
    past the caption length rounded up to the sequence multiple, with (row, column) on the other two axes."""
    padded = -(-cap_len // SEQ_MULTIPLE) * SEQ_MULTIPLE
    img = torch.zeros(h_tokens, w_tokens, 3, device=device)
    img[..., 0] = padded + 1
    img[..., 1] = torch.arange(h_tokens, device=device)[:, None]
    img[..., 2] = torch.arange(w_tokens, device=device)[None, :]
    cap = torch.zeros(cap_len, 3, device=device)
    cap[:, 0] = torch.arange(1, cap_len + 1, device=device)
    return img.reshape(-1, 3), cap


def timestep_features(t: torch.Tensor, scale: float) -> torch.Tensor:
    """[B] -> [B, 256]: cos block then sin block of t * scale at 128 log-spaced frequencies."""
    half = 128
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = (t.float() * scale)[:, None] * freqs[None]
    return torch.cat([a.cos(), a.sin()], -1)


def _rope_pairs(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, heads, hd], cos/sin [S, hd/2]: rotation of consecutive pairs."""
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), -1).flatten(-2)


class OracleZImageDiT:
    def __init__(self, cfg: ZImageConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
        self.dtype, self.device = dtype, torch.device(device)
        self.lora = None                    # training: {module name: (A [r, in], B [out, r], scale)}

    def _lin(self, x, name):
        y = F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))
        if self.lora is not None and name in self.lora:
            y = y + adapter_residual(self.lora[name], x)
        return y

    def _rms(self, x, name, eps=None):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + (eps or self.cfg.norm_eps))
        return (y * self.w[name + ".weight"].float()).to(x.dtype)

    def _attention(self, x, p, cos, sin):
        cfg = self.cfg
        B, S, _ = x.shape
        q, k, v = (self._lin(x, f"{p}.attention.{n}").view(B, S, cfg.n_heads, cfg.head_dim)
                   for n in ("to_q", "to_k", "to_v"))
        q = _rope_pairs(self._rms(q, f"{p}.attention.norm_q", 1e-5), cos, sin)
        k = _rope_pairs(self._rms(k, f"{p}.attention.norm_k", 1e-5), cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return self._lin(o.transpose(1, 2).reshape(B, S, -1), f"{p}.attention.to_out.0")

    def _ffn(self, x, p):
        return self._lin(F.silu(self._lin(x, f"{p}.feed_forward.w1")) * self._lin(x, f"{p}.feed_forward.w3"),
                         f"{p}.feed_forward.w2")

    def _block(self, x, p, cos, sin, adaln):
        if adaln is not None:
            sa, ga, sm, gm = self._lin(adaln, f"{p}.adaLN_modulation.0")[:, None, :].chunk(4, -1)
            sa, sm, ga, gm = 1 + sa, 1 + sm, ga.tanh(), gm.tanh()
        else:
            sa = sm = ga = gm = 1.0
        a = self._attention(self._rms(x, f"{p}.attention_norm1") * sa, p, cos, sin)
        x = x + ga * self._rms(a, f"{p}.attention_norm2")
        f = self._ffn(self._rms(x, f"{p}.ffn_norm1") * sm, p)
        return x + gm * self._rms(f, f"{p}.ffn_norm2")

    def refine_caption(self, cap_feats: torch.Tensor) -> torch.Tensor:
        """[B, L, cap_feat_dim] -> caption tokens [B, L, dim] (no dependence on the timestep)."""
        cfg = self.cfg
        cap = self._lin(self._rms(cap_feats.to(self.device, self.dtype), "cap_embedder.0"), "cap_embedder.1")
        _, cap_ids = position_ids(1, 1, cap.shape[1], self.device)
        cos, sin = rope_table(cap_ids, cfg.axes_dims, cfg.rope_theta)
        for i in range(cfg.n_refiner_layers):
            cap = self._block(cap, f"context_refiner.{i}", cos, sin, None)
        return cap

    def forward_grad(self, z: torch.Tensor, t: torch.Tensor, cap_feats: torch.Tensor) -> torch.Tensor:
        """z [B, C, H, W] latent, t [B] in [0, 1] (1 - sigma), cap_feats [B, L, cap_feat_dim] -> [B, C, H, W]."""
        cfg = self.cfg
        B, _, H, W = z.shape
        p = cfg.patch_size
        adaln = self._lin(F.silu(self._lin(timestep_features(t.to(self.device), cfg.t_scale).to(self.dtype),
                                           "t_embedder.mlp.0")), "t_embedder.mlp.2")
        x = self._lin(patchify(z.to(self.device, self.dtype), p), "all_x_embedder.2-1")
        cap = self.refine_caption(cap_feats)
        img_ids, cap_ids = position_ids(H // p, W // p, cap.shape[1], self.device)
        cos_i, sin_i = rope_table(img_ids, cfg.axes_dims, cfg.rope_theta)
        for i in range(cfg.n_refiner_layers):
            x = self._block(x, f"noise_refiner.{i}", cos_i, sin_i, adaln)
        cos, sin = rope_table(torch.cat([img_ids, cap_ids], 0), cfg.axes_dims, cfg.rope_theta)
        n_img = x.shape[1]
        u = torch.cat([x, cap], 1)
        for i in range(cfg.n_layers):
            u = self._block(u, f"layers.{i}", cos, sin, adaln)
        scale = 1 + self._lin(F.silu(adaln), "all_final_layer.2-1.adaLN_modulation.1")
        out = self._lin(F.layer_norm(u[:, :n_img], (cfg.dim,), eps=1e-6) * scale[:, None, :],
                        "all_final_layer.2-1.linear")
        return unpatchify(out, H, W, p)

    @torch.no_grad()
    def forward(self, z, t, cap_feats):
        return self.forward_grad(z, t, cap_feats)


# =================================================================================================================
# sm_100a model
# =================================================================================================================
class ZImageDiTGpu:
    """One image per forward (classifier-free guidance runs two forwards, their captions differ in length)."""

    def __init__(self, cfg: ZImageConfig, device: torch.device | None = None):
        assert cfg.head_dim == 128, "the sm_100a attention kernels are built for head_dim 128"
        self.cfg = cfg
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.w: dict[str, torch.Tensor] = {}
        self.launches = 0

    def load_state_dict(self, weights: dict[str, torch.Tensor]) -> "ZImageDiTGpu":
        cfg = self.cfg
        dev = self.device
        w = {k: v.to(device=dev, dtype=torch.bfloat16).contiguous() for k, v in weights.items()
             if k not in ("x_pad_token", "cap_pad_token")}
        mod_w, mod_b, norms = [], [], {n: [] for n in ("attention_norm1", "ffn_norm1")}
        self._mod_index: dict[str, int] = {}
        for p, modulated in block_names(cfg):
            a = f"{p}.attention."
            w[a + "qkv.weight"] = torch.cat([w.pop(a + f"{n}.weight") for n in ("to_q", "to_k", "to_v")], 0).contiguous()
            w1, w3 = w.pop(f"{p}.feed_forward.w1.weight"), w.pop(f"{p}.feed_forward.w3.weight")
            w[f"{p}.feed_forward.w13.weight"] = torch.stack([w1, w3], 1).reshape(-1, w1.shape[1]).contiguous()
            if modulated:
                self._mod_index[p] = len(mod_w)
                mod_w.append(w.pop(f"{p}.adaLN_modulation.0.weight"))
                mod_b.append(w.pop(f"{p}.adaLN_modulation.0.bias"))
                for n in norms:
                    norms[n].append(w[f"{p}.{n}.weight"].float())
        # every modulation linear reads the same 256-wide vector: one GEMM per step for all blocks and the final layer
        self._mod_w = torch.cat(mod_w + [w.pop("all_final_layer.2-1.adaLN_modulation.1.weight")], 0).contiguous()
        self._mod_b = torch.cat(mod_b + [w.pop("all_final_layer.2-1.adaLN_modulation.1.bias")], 0).contiguous()
        self._norm1 = torch.stack(norms["attention_norm1"], 0)            # [blocks, dim] fp32
        self._norm3 = torch.stack(norms["ffn_norm1"], 0)
        self.w = w
        return self

    def init_random(self, seed: int = 0, std: float = 0.02) -> "ZImageDiTGpu":
        return self.load_state_dict(random_zimage_weights(self.cfg, seed, std, torch.bfloat16, self.device))

    def weight_bytes(self) -> int:
        return sum(t.numel() * 2 for t in self.w.values()) + self._mod_w.numel() * 2

    # ---- pieces ------------------------------------------------------------------------------------------------
    def _lin(self, x, name, **kw):
        from .. import ops

        self.launches += 1
        return ops.gemm_bf16(x, self.w[name + ".weight"], bias=self.w.get(name + ".bias"), **kw)

    def _block(self, x, p, positions, cos, sin, mods):
        """x [S, dim] bf16. mods: None, or (norm1 weights * (1 + scale_msa), tanh(gate_msa), norm3 weights *
        (1 + scale_mlp), tanh(gate_mlp)), each [dim] bf16."""
        from .. import ops

        cfg = self.cfg
        S, D = x.shape
        NH, HD, eps = cfg.n_heads, cfg.head_dim, cfg.norm_eps
        w = self.w
        n1 = mods[0] if mods else w[f"{p}.attention_norm1.weight"]
        n3 = mods[2] if mods else w[f"{p}.ffn_norm1.weight"]
        qkv = self._lin(ops.rmsnorm(x, n1, eps), f"{p}.attention.qkv")
        ops.rope_kv_write(qkv, positions, None, cos, sin, None, None, NH, NH, HD, rot_dim=HD, interleaved=True,
                          q_norm=w[f"{p}.attention.norm_q.weight"], k_norm=w[f"{p}.attention.norm_k.weight"],
                          norm_eps=1e-5)
        q3 = qkv.view(1, S, 3 * NH, HD)
        attn = ops.dense_attention(q3[:, :, :NH], q3[:, :, NH:2 * NH], q3[:, :, 2 * NH:], scale=HD ** -0.5)
        a = ops.rmsnorm(self._lin(attn.view(S, D), f"{p}.attention.to_out.0"), w[f"{p}.attention_norm2.weight"], eps)
        x = ops.gated_residual(x, a, mods[1] if mods else None)
        h = ops.linear_gated(ops.rmsnorm(x, n3, eps), w[f"{p}.feed_forward.w13.weight"])
        f = ops.rmsnorm(self._lin(h, f"{p}.feed_forward.w2"), w[f"{p}.ffn_norm2.weight"], eps)
        self.launches += 9
        return ops.gated_residual(x, f, mods[3] if mods else None)

    @torch.no_grad()
    def refine_caption(self, cap_feats: torch.Tensor) -> torch.Tensor:
        """[1, L, cap_feat_dim] -> caption tokens [L, dim]; computed once per prompt."""
        from .. import ops

        cfg = self.cfg
        c = cap_feats.to(self.device, torch.bfloat16).reshape(-1, cfg.cap_feat_dim).contiguous()
        cap = self._lin(ops.rmsnorm(c, self.w["cap_embedder.0.weight"], cfg.norm_eps), "cap_embedder.1")
        L = cap.shape[0]
        _, ids = position_ids(1, 1, L, self.device)
        cos, sin = rope_table(ids, cfg.axes_dims, cfg.rope_theta)
        pos = torch.arange(L, dtype=torch.int32, device=self.device)
        for i in range(cfg.n_refiner_layers):
            cap = self._block(cap, f"context_refiner.{i}", pos, cos, sin, None)
        return cap

    def rope_tables(self, h_tokens: int, w_tokens: int, cap_len: int):
        cfg = self.cfg
        img_ids, cap_ids = position_ids(h_tokens, w_tokens, cap_len, self.device)
        return (rope_table(img_ids, cfg.axes_dims, cfg.rope_theta),
                rope_table(torch.cat([img_ids, cap_ids], 0), cfg.axes_dims, cfg.rope_theta))

    def _modulations(self, t: torch.Tensor):
        """t [1] -> per modulated block the four per-step vectors, and the final layer's (1 + scale)."""
        from .. import ops

        cfg = self.cfg
        D = cfg.dim
        feat = timestep_features(t.to(self.device), cfg.t_scale).bfloat16()
        adaln = self._lin(self._lin(feat, "t_embedder.mlp.0", act="silu"), "t_embedder.mlp.2")        # [1, 256]
        nb = len(self._mod_index)
        # rows [0, nb * 4D) take the vector itself, the final layer's rows take silu of it: two GEMMs on row ranges
        blocks = ops.gemm_bf16(adaln, self._mod_w[: nb * 4 * D], bias=self._mod_b[: nb * 4 * D]).view(nb, 4, D).float()
        fin = ops.gemm_bf16(F.silu(adaln.float()).bfloat16(), self._mod_w[nb * 4 * D:], bias=self._mod_b[nb * 4 * D:])
        self.launches += 2
        n1 = (self._norm1 * (1 + blocks[:, 0])).bfloat16()
        n3 = (self._norm3 * (1 + blocks[:, 2])).bfloat16()
        gates = blocks[:, 1::2].tanh().bfloat16()          # rows 1 and 3: the two gates
        return n1, gates[:, 0].contiguous(), n3, gates[:, 1].contiguous(), fin

    @torch.no_grad()
    def forward(self, z: torch.Tensor, t: torch.Tensor, cap_tokens: torch.Tensor, ropes=None) -> torch.Tensor:
        """z [1, C, H, W], t [1] (1 - sigma), cap_tokens = refine_caption(...) -> velocity [1, C, H, W] bf16."""
        from .. import ops

        cfg = self.cfg
        _, _, H, W = z.shape
        p = cfg.patch_size
        self.launches = 0
        L = cap_tokens.shape[0]
        (cos_i, sin_i), (cos, sin) = ropes if ropes is not None else self.rope_tables(H // p, W // p, L)
        n1, g1, n3, g3, fin = self._modulations(t)
        x = self._lin(patchify(z.to(self.device, torch.bfloat16), p)[0].contiguous(), "all_x_embedder.2-1")
        n_img = x.shape[0]
        pos = torch.arange(n_img + L, dtype=torch.int32, device=self.device)

        def mods(pfx):
            i = self._mod_index[pfx]
            return n1[i], g1[i], n3[i], g3[i]
        for i in range(cfg.n_refiner_layers):
            x = self._block(x, f"noise_refiner.{i}", pos[:n_img], cos_i, sin_i, mods(f"noise_refiner.{i}"))
        u = torch.cat([x, cap_tokens], 0)
        for i in range(cfg.n_layers):
            u = self._block(u, f"layers.{i}", pos, cos, sin, mods(f"layers.{i}"))
        out = self._lin(ops.layernorm_mod(u[:n_img], scale=fin, eps=1e-6),
                        "all_final_layer.2-1.linear")
        self.launches += 1
        return unpatchify(out[None], H, W, p)

    def forward_graphed(self, z, t, cap_tokens, ropes=None):
        """Same result as forward(); the first call for a shape captures a CUDA graph, later calls replay it."""
        key = (tuple(z.shape), tuple(cap_tokens.shape))
        st = self.__dict__.setdefault("_graphs", {})
        g = st.get(key)
        if g is None:
            if ropes is None:
                ropes = self.rope_tables(z.shape[2] // self.cfg.patch_size, z.shape[3] // self.cfg.patch_size,
                                         cap_tokens.shape[0])
            static = {"z": z.to(self.device, torch.bfloat16).clone(), "t": t.to(self.device).float().clone(),
                      "cap": cap_tokens.clone()}         # the caption is an input like the others: one graph per shape
            run = lambda: self.forward(static["z"], static["t"], static["cap"], ropes)      # noqa: E731
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static["out"] = run()
            static["launches"] = self.launches
            g = st[key] = (graph, static)
        graph, static = g
        static["z"].copy_(z)
        static["t"].copy_(t)
        static["cap"].copy_(cap_tokens)
        graph.replay()
        self.launches = static["launches"]
        return static["out"]
