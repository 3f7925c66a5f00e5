"""FLUX-style rectified-flow DiT: an fp32 PyTorch oracle and the sm_100a model.

Architecture (parity target: candle-gen-flux/src/ip_dit.rs:404-547,719-815): img_in / txt_in projections; vec =
time_in(temb(1000 t)) + guidance_in(temb(1000 g)) + vector_in(pooled); 3-axis RoPE table from (txt_ids, img_ids);
N_double double-stream blocks (separate img / txt weights, joint attention over cat(txt, img)) and N_single
single-stream blocks (fused qkv + MLP linear1, linear2 over cat(attn, gelu(mlp))); adaLN final layer.

The GPU model never concatenates: both streams' QKV GEMMs write into row ranges of one joint [S, 3*H*D] buffer,
the attention kernel writes into the first columns of the single-block linear2 input whose remaining columns are
written by the MLP GEMM with a fused tanh-GELU epilogue, QK-RMSNorm and RoPE run in place in one kernel, and
adaLN modulation / gated residuals are fused kernels."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .nn_dual import adapter_residual

from .. import ops
from ..parallel.comm import Communicator, single


@dataclass
class FluxConfig:
    in_channels: int = 64
    vec_in_dim: int = 768
    context_in_dim: int = 4096
    hidden_size: int = 3072
    mlp_ratio: float = 4.0
    num_heads: int = 24
    depth: int = 19
    depth_single: int = 38
    axes_dim: tuple[int, int, int] = (16, 56, 56)
    theta: float = 10000.0
    guidance_embed: bool = True

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)

    @staticmethod
    def tiny() -> "FluxConfig":
        return FluxConfig(in_channels=16, vec_in_dim=32, context_in_dim=64, hidden_size=256, num_heads=2, depth=2,
                          depth_single=2, axes_dim=(16, 56, 56))


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0, time_factor: float = 1000.0
                       ) -> torch.Tensor:
    t = time_factor * t.float()
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rope_table(ids: torch.Tensor, axes_dim, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [S, 3] -> (cos, sin) [S, sum(axes_dim) / 2] for interleaved-pair rotation."""
    cos, sin = [], []
    for i, d in enumerate(axes_dim):
        omega = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        ang = ids[:, i].double()[:, None] * omega[None]
        cos.append(ang.cos())
        sin.append(ang.sin())
    return torch.cat(cos, -1).float().contiguous(), torch.cat(sin, -1).float().contiguous()


def make_ids(h_tokens: int, w_tokens: int, txt_len: int, device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    img = torch.zeros(h_tokens, w_tokens, 3, device=device)
    img[..., 1] = torch.arange(h_tokens, device=device)[:, None]
    img[..., 2] = torch.arange(w_tokens, device=device)[None, :]
    return torch.zeros(txt_len, 3, device=device), img.reshape(-1, 3)


def random_flux_weights(cfg: FluxConfig, seed: int = 0, std: float = 0.02, dtype=torch.float32, device="cpu"
                        ) -> dict[str, torch.Tensor]:
    g = torch.Generator(device=device).manual_seed(seed)
    H, M = cfg.hidden_size, cfg.mlp_hidden
    w: dict[str, torch.Tensor] = {}

    def lin(name, out_f, in_f):
        w[name + ".weight"] = (torch.randn(out_f, in_f, generator=g, device=device) * std).to(dtype)
        w[name + ".bias"] = (torch.randn(out_f, generator=g, device=device) * std).to(dtype)

    lin("img_in", H, cfg.in_channels)
    lin("txt_in", H, cfg.context_in_dim)
    for n, d in (("time_in", 256), ("vector_in", cfg.vec_in_dim), ("guidance_in", 256)):
        if n == "guidance_in" and not cfg.guidance_embed:
            continue
        lin(f"{n}.in_layer", H, d)
        lin(f"{n}.out_layer", H, H)
    ones = lambda: (torch.ones(cfg.head_dim, device=device) + 0.1 * torch.randn(cfg.head_dim, generator=g, device=device)).to(dtype)  # noqa: E731
    for i in range(cfg.depth):
        for s in ("img", "txt"):
            p = f"double_blocks.{i}.{s}"
            lin(f"{p}_mod.lin", 6 * H, H)
            lin(f"{p}_attn.qkv", 3 * H, H)
            w[f"{p}_attn.norm.query_norm.scale"] = ones()
            w[f"{p}_attn.norm.key_norm.scale"] = ones()
            lin(f"{p}_attn.proj", H, H)
            lin(f"{p}_mlp.0", M, H)
            lin(f"{p}_mlp.2", H, M)
    for i in range(cfg.depth_single):
        p = f"single_blocks.{i}"
        lin(f"{p}.modulation.lin", 3 * H, H)
        lin(f"{p}.linear1", 3 * H + M, H)
        lin(f"{p}.linear2", H, H + M)
        w[f"{p}.norm.query_norm.scale"] = ones()
        w[f"{p}.norm.key_norm.scale"] = ones()
    lin("final_layer.adaLN_modulation.1", 2 * H, H)
    lin("final_layer.linear", cfg.in_channels, H)
    return w


# =================================================================================================================
# fp32 oracle
# =================================================================================================================
class OracleFluxDiT:
    def __init__(self, cfg: FluxConfig, weights: dict[str, torch.Tensor], dtype=torch.float32, device="cpu"):
        self.cfg = cfg
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}

    lora: dict | None = None     # {module name: (A [r, in], B [out, r], scale)}: low-rank deltas added on the fly

    def _lin(self, x, name):
        y = F.linear(x, self.w[name + ".weight"], self.w[name + ".bias"])
        if self.lora is not None and name in self.lora:
            y = y + adapter_residual(self.lora[name], x)
        return y

    def _mlp_embed(self, x, name):
        return self._lin(F.silu(self._lin(x, name + ".in_layer")), name + ".out_layer")

    @staticmethod
    def _rms(x, scale, eps=1e-6):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * scale

    @staticmethod
    def _rope(x, cos, sin):
        # x [B, S, H, D]; interleaved pairs
        x0, x1 = x[..., 0::2], x[..., 1::2]
        c, s = cos[None, :, None, :].to(x.dtype), sin[None, :, None, :].to(x.dtype)
        return torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1).flatten(-2)

    def _attn(self, q, k, v, cos, sin):
        q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return o.transpose(1, 2).flatten(-2)

    def _qkv(self, x, prefix, norm_prefix):
        B, S, _ = x.shape
        H, D = self.cfg.num_heads, self.cfg.head_dim
        q, k, v = x.view(B, S, 3, H, D).unbind(2)
        return (self._rms(q, self.w[norm_prefix + ".query_norm.scale"]),
                self._rms(k, self.w[norm_prefix + ".key_norm.scale"]), v)

    @torch.no_grad()
    def forward(self, img, img_ids, txt, txt_ids, timesteps, y, guidance=None):
        return self.forward_grad(img, img_ids, txt, txt_ids, timesteps, y, guidance)

    def _modulations(self, timesteps, y, guidance, dtype) -> dict[str, torch.Tensor]:
        """{modulation name: [B, rows]}: every adaLN modulation is a linear map of silu(conditioning vector)."""
        cfg = self.cfg
        vec = self._mlp_embed(timestep_embedding(timesteps).to(dtype), "time_in")
        if cfg.guidance_embed:
            vec = vec + self._mlp_embed(timestep_embedding(guidance).to(dtype), "guidance_in")
        vec = vec + self._mlp_embed(y, "vector_in")
        sv = F.silu(vec)
        names = [f"double_blocks.{i}.{s}_mod.lin" for i in range(cfg.depth) for s in ("img", "txt")]
        names += [f"single_blocks.{i}.modulation.lin" for i in range(cfg.depth_single)]
        return {n: self._lin(sv, n) for n in names + ["final_layer.adaLN_modulation.1"]}

    def forward_grad(self, img, img_ids, txt, txt_ids, timesteps, y, guidance=None):
        """The same computation with autograd enabled (adapter training differentiates through it)."""
        cfg = self.cfg
        Hs = cfg.hidden_size
        cos, sin = rope_table(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.theta)
        img = self._lin(img, "img_in")
        txt = self._lin(txt, "txt_in")
        M = self._modulations(timesteps, y, guidance, img.dtype)
        ln = lambda x: F.layer_norm(x, (Hs,), eps=1e-6)  # noqa: E731
        T = txt.shape[1]
        inj = getattr(self, "injector", None)      # image-stream residual hooks (identity adapters): see FluxDiTGpu.injector
        for i in range(cfg.depth):
            mods = {}
            for s in ("img", "txt"):
                mods[s] = M[f"double_blocks.{i}.{s}_mod.lin"][:, None, :].chunk(6, dim=-1)
            qkvs = {}
            for s, x in (("img", img), ("txt", txt)):
                sh1, sc1 = mods[s][0], mods[s][1]
                xm = (1 + sc1) * ln(x) + sh1
                qkvs[s] = self._qkv(self._lin(xm, f"double_blocks.{i}.{s}_attn.qkv"), None,
                                    f"double_blocks.{i}.{s}_attn.norm")
            if inj is not None and hasattr(inj, "on_img_query"):
                inj.on_img_query(i, qkvs["img"][0])          # [B, S_img, heads, head_dim]: after the q norm, before rotation
            q = torch.cat([qkvs["txt"][0], qkvs["img"][0]], 1)
            k = torch.cat([qkvs["txt"][1], qkvs["img"][1]], 1)
            v = torch.cat([qkvs["txt"][2], qkvs["img"][2]], 1)
            attn = self._attn(q, k, v, cos, sin)
            outs = {}
            for s, x, a in (("img", img, attn[:, T:]), ("txt", txt, attn[:, :T])):
                _, _, g1, sh2, sc2, g2 = mods[s]
                x = x + g1 * self._lin(a, f"double_blocks.{i}.{s}_attn.proj")
                h = (1 + sc2) * ln(x) + sh2
                h = self._lin(F.gelu(self._lin(h, f"double_blocks.{i}.{s}_mlp.0"), approximate="tanh"),
                              f"double_blocks.{i}.{s}_mlp.2")
                outs[s] = x + g2 * h
            img, txt = outs["img"], outs["txt"]
            r = inj.after_double(i, img) if inj is not None else None
            if r is not None:
                img = img + r.to(img.dtype)
        x = torch.cat([txt, img], 1)
        for i in range(cfg.depth_single):
            p = f"single_blocks.{i}"
            sh, sc, g = M[p + ".modulation.lin"][:, None, :].chunk(3, dim=-1)
            xm = (1 + sc) * ln(x) + sh
            l1 = self._lin(xm, p + ".linear1")
            qkv, mlp = l1[..., : 3 * Hs], l1[..., 3 * Hs:]
            q, k, v = self._qkv(qkv, None, p + ".norm")
            attn = self._attn(q, k, v, cos, sin)
            x = x + g * self._lin(torch.cat([attn, F.gelu(mlp, approximate="tanh")], -1), p + ".linear2")
            r = inj.after_single(i, x[:, T:]) if inj is not None else None
            if r is not None:
                x = torch.cat([x[:, :T], x[:, T:] + r.to(x.dtype)], 1)
        img = x[:, T:]
        sh, sc = M["final_layer.adaLN_modulation.1"][:, None, :].chunk(2, dim=-1)
        return self._lin((1 + sc) * ln(img) + sh, "final_layer.linear")


# =================================================================================================================
# sm_100a model
# =================================================================================================================
class FluxDiTGpu:
    def __init__(self, cfg: FluxConfig, comm: Communicator | None = None, device: torch.device | None = None):
        assert cfg.head_dim == 128, "the sm_100a attention kernels are built for head_dim 128"
        self.cfg = cfg
        self.comm = comm or single(device)
        self.device = device or self.comm.device
        self.w: dict[str, torch.Tensor] = {}
        self.launches = 0
        # Optional image-stream hooks (candle-gen-flux `DitImageInjector`): an object with after_double(i, img) and
        # after_single(i, img_tokens), each returning a residual [B, S_img, hidden] or None. Single-GPU eager path only.
        self.injector = None

    def load_state_dict(self, weights: dict[str, torch.Tensor]) -> "FluxDiTGpu":
        self.w = {k: v.to(device=self.device, dtype=torch.bfloat16).contiguous() for k, v in weights.items()}
        H = self.cfg.hidden_size
        # split single-block linear1 into its qkv and MLP row blocks so the MLP part takes the fused GELU epilogue
        for i in range(self.cfg.depth_single):
            p = f"single_blocks.{i}.linear1"
            W, b = self.w.pop(p + ".weight"), self.w.pop(p + ".bias")
            self.w[p + "_qkv.weight"], self.w[p + "_mlp.weight"] = W[: 3 * H].contiguous(), W[3 * H:].contiguous()
            self.w[p + "_qkv.bias"], self.w[p + "_mlp.bias"] = b[: 3 * H].contiguous(), b[3 * H:].contiguous()
        self._build_modulation_table()
        return self

    def _mod_names(self) -> list[str]:
        names = []
        for i in range(self.cfg.depth):
            names += [f"double_blocks.{i}.img_mod.lin", f"double_blocks.{i}.txt_mod.lin"]
        names += [f"single_blocks.{i}.modulation.lin" for i in range(self.cfg.depth_single)]
        return names + ["final_layer.adaLN_modulation.1"]

    def _build_modulation_table(self) -> None:
        """Every adaLN modulation is a linear map of the same conditioning vector, so all of them (344 x hidden output
        rows for FLUX.1) are one GEMM per step. The per-block weights become views into the concatenated matrix; with
        a parallel communicator each rank computes a contiguous share of the rows and the shares are all-gathered."""
        names = self._mod_names()
        sizes = [self.w[n + ".weight"].shape[0] for n in names]
        total = sum(sizes)
        P = self.comm.world
        pad = (-total) % (8 * P)
        big_w = torch.empty((total + pad, self.cfg.hidden_size), dtype=torch.bfloat16, device=self.device)
        big_b = torch.zeros(total + pad, dtype=torch.bfloat16, device=self.device)
        off = 0
        self._mod_slices = {}
        for n, sz in zip(names, sizes):
            big_w[off:off + sz].copy_(self.w.pop(n + ".weight"))
            big_b[off:off + sz].copy_(self.w.pop(n + ".bias"))
            self.w[n + ".weight"], self.w[n + ".bias"] = big_w[off:off + sz], big_b[off:off + sz]
            self._mod_slices[n] = (off, sz)
            off += sz
        if pad:
            big_w[total:].zero_()
        self._mod_w, self._mod_b = big_w, big_b

    def _all_modulations(self, sv: torch.Tensor) -> dict[str, torch.Tensor]:
        """sv [B, H] -> {modulation name: [B, rows]} from one GEMM (plus an all-gather when parallel)."""
        P, r = self.comm.world, self.comm.rank
        n = self._mod_w.shape[0] // P
        out = ops.gemm_bf16(sv, self._mod_w[r * n:(r + 1) * n], bias=self._mod_b[r * n:(r + 1) * n])
        self.launches += 1
        if P > 1:
            out = self.comm.all_gather(out, dim=1)
        return {name: out[:, off:off + sz] for name, (off, sz) in self._mod_slices.items()}

    def init_random(self, seed: int = 0, std: float = 0.02) -> "FluxDiTGpu":
        return self.load_state_dict(random_flux_weights(self.cfg, seed, std, torch.bfloat16, self.device))

    def weight_bytes(self) -> int:
        return sum(t.numel() * 2 for t in self.w.values())

    def _lin(self, x, name, **kw):
        self.launches += 1
        return ops.gemm_bf16(x, self.w[name + ".weight"], bias=self.w[name + ".bias"], **kw)

    def _embed(self, x, name):
        return self._lin(self._lin(x, name + ".in_layer", act="silu"), name + ".out_layer")

    def conditioning_vector(self, timesteps, y, guidance) -> torch.Tensor:
        vec = self._embed(timestep_embedding(timesteps).bfloat16(), "time_in")
        if self.cfg.guidance_embed:
            vec = vec + self._embed(timestep_embedding(guidance).bfloat16(), "guidance_in")
        vec = vec + self._embed(y.bfloat16(), "vector_in")
        return F.silu(vec.float()).bfloat16().contiguous()   # [B, H]: silu(vec), the input of every modulation

    @torch.no_grad()
    def forward(self, img, img_ids, txt, txt_ids, timesteps, y, guidance=None, rope=None):
        """img [B, S_img, C_in], txt [B, S_txt, C_ctx] bf16 -> velocity [B, S_img, C_in] bf16. With a parallel
        communicator every rank passes the full inputs and receives the full velocity; the work in between is
        sequence-parallel (each rank owns 1/P of the text and of the image tokens, and 1/P of the heads inside
        attention)."""
        if self.comm.world > 1:
            return self._forward_sp(img, img_ids, txt, txt_ids, timesteps, y, guidance, rope)
        cfg = self.cfg
        H, D, NH, M = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.mlp_hidden
        B, Si, _ = img.shape
        St = txt.shape[1]
        S = St + Si
        dev = img.device
        self.launches = 0
        if rope is None:
            rope = rope_table(torch.cat([txt_ids, img_ids], 0).to(dev), cfg.axes_dim, cfg.theta)
        cos, sin = rope
        positions = torch.arange(S, dtype=torch.int32, device=dev).repeat(B)
        sv = self.conditioning_vector(timesteps, y, guidance)
        mod = self._all_modulations(sv)
        x_img = self._lin(img.reshape(B * Si, -1), "img_in").view(B, Si, H)
        x_txt = self._lin(txt.reshape(B * St, -1), "txt_in").view(B, St, H)
        scale = D ** -0.5
        inj = self.injector
        qkv = torch.empty((B, S, 3 * H), dtype=torch.bfloat16, device=dev)
        attn = torch.empty((B, S, H), dtype=torch.bfloat16, device=dev)

        def attention(qkv_buf, out_buf):
            w = self._cur_norm
            ops.rope_kv_write(qkv_buf.view(B * S, 3 * H), positions, None, cos, sin, None, None, NH, NH, D,
                              rot_dim=D, interleaved=True, q_norm=w[0], k_norm=w[1], norm_eps=1e-6)
            q = qkv_buf[:, :, :H].unflatten(-1, (NH, D))
            k = qkv_buf[:, :, H:2 * H].unflatten(-1, (NH, D))
            v = qkv_buf[:, :, 2 * H:].unflatten(-1, (NH, D))
            ops.dense_attention(q, k, v, scale=scale, out=out_buf)
            self.launches += 2

        for i in range(cfg.depth):
            mods = {}
            for s in ("img", "txt"):
                m = mod[f"double_blocks.{i}.{s}_mod.lin"]                      # [B, 6H]
                mods[s] = [m[:, j * H:(j + 1) * H] for j in range(6)]
            for s, x, lo, n in (("txt", x_txt, 0, St), ("img", x_img, St, Si)):
                xm = ops.layernorm_mod(x, scale=mods[s][1], shift=mods[s][0], rows_per_batch=n)
                for b in range(B):
                    self._lin(xm[b], f"double_blocks.{i}.{s}_attn.qkv", out=qkv[b, lo:lo + n])
                self.launches += 1
            if inj is not None and hasattr(inj, "on_img_query"):
                # adapters that attend from the image query want it after the q norm and before rotation; the fused
                # norm + rotation below works in place, so this copy is normalised on its own
                inj.on_img_query(i, ops.rmsnorm(qkv[:, St:, :H].reshape(B * Si * NH, D).contiguous(),
                                                self.w[f"double_blocks.{i}.img_attn.norm.query_norm.scale"], 1e-6)
                                 .view(B, Si, NH, D))
            # per-stream QK norms differ: rotate each row range with its own norm weights
            for s, lo, n in (("txt", 0, St), ("img", St, Si)):
                nw = (self.w[f"double_blocks.{i}.{s}_attn.norm.query_norm.scale"],
                      self.w[f"double_blocks.{i}.{s}_attn.norm.key_norm.scale"])
                for b in range(B):
                    ops.rope_kv_write(qkv[b, lo:lo + n], positions[lo:lo + n], None, cos, sin, None, None, NH, NH, D,
                                      rot_dim=D, interleaved=True, q_norm=nw[0], k_norm=nw[1], norm_eps=1e-6)
                    self.launches += 1
            q = qkv[:, :, :H].unflatten(-1, (NH, D))
            k = qkv[:, :, H:2 * H].unflatten(-1, (NH, D))
            v = qkv[:, :, 2 * H:].unflatten(-1, (NH, D))
            ops.dense_attention(q, k, v, scale=scale, out=attn)
            self.launches += 1
            new = {}
            for s, x, lo, n in (("txt", x_txt, 0, St), ("img", x_img, St, Si)):
                a = attn[:, lo:lo + n]
                proj = torch.empty((B, n, H), dtype=torch.bfloat16, device=dev)
                for b in range(B):
                    self._lin(a[b], f"double_blocks.{i}.{s}_attn.proj", out=proj[b])
                x = ops.gated_residual(x, proj, mods[s][2], rows_per_batch=n)
                hm = ops.layernorm_mod(x, scale=mods[s][4], shift=mods[s][3], rows_per_batch=n)
                h1 = self._lin(hm.view(B * n, H), f"double_blocks.{i}.{s}_mlp.0", act="gelu_tanh")
                h2 = self._lin(h1, f"double_blocks.{i}.{s}_mlp.2").view(B, n, H)
                new[s] = ops.gated_residual(x, h2, mods[s][5], rows_per_batch=n)
                self.launches += 3
            x_img, x_txt = new["img"], new["txt"]
            r = inj.after_double(i, x_img) if inj is not None else None
            if r is not None:
                x_img = x_img + r.to(x_img.dtype)

        x = torch.cat([x_txt, x_img], 1).contiguous()
        buf2 = torch.empty((B, S, H + M), dtype=torch.bfloat16, device=dev)
        for i in range(cfg.depth_single):
            p = f"single_blocks.{i}"
            m = mod[p + ".modulation.lin"]
            sh, sc, g = m[:, :H], m[:, H:2 * H], m[:, 2 * H:]
            xm = ops.layernorm_mod(x, scale=sc, shift=sh, rows_per_batch=S).view(B * S, H)
            self._lin(xm, p + ".linear1_qkv", out=qkv.view(B * S, 3 * H))
            self._lin(xm, p + ".linear1_mlp", act="gelu_tanh", out=buf2.view(B * S, H + M)[:, H:])
            self._cur_norm = (self.w[p + ".norm.query_norm.scale"], self.w[p + ".norm.key_norm.scale"])
            attention(qkv, buf2[:, :, :H])
            out = self._lin(buf2.view(B * S, H + M), p + ".linear2").view(B, S, H)
            x = ops.gated_residual(x, out, g, rows_per_batch=S)
            self.launches += 2
            r = inj.after_single(i, x[:, St:]) if inj is not None else None
            if r is not None:
                x[:, St:] += r.to(x.dtype)
        x_img = x[:, St:].contiguous()
        m = mod["final_layer.adaLN_modulation.1"]
        xm = ops.layernorm_mod(x_img, scale=m[:, H:], shift=m[:, :H], rows_per_batch=Si)
        self.launches += 1
        return self._lin(xm.view(B * Si, H), "final_layer.linear").view(B, Si, -1)

    # ---------------------------------------------------------------------------------------------------------
    # CUDA-graph replay (the forward has static shapes: one capture per (image tokens, text tokens) pair)
    # ---------------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_graphed(self, img, img_ids, txt, txt_ids, timesteps, y, guidance=None, rope=None):
        """Same result as forward(); the first call for a shape runs eagerly once (allocations, tensor maps,
        symmetric-memory rendezvous) and captures, later calls copy the inputs into static buffers and replay."""
        if self.injector is not None:           # the hooks read per-request tensors: no capture
            return self.forward(img, img_ids, txt, txt_ids, timesteps, y, guidance, rope)
        key = (tuple(img.shape), tuple(txt.shape), guidance is not None)
        st = getattr(self, "_graphs", None)
        if st is None:
            st = self._graphs = {}
        g = st.get(key)
        if g is None:
            if rope is None:
                rope = rope_table(torch.cat([txt_ids, img_ids], 0).to(img.device), self.cfg.axes_dim, self.cfg.theta)
            static = {"img": img.clone(), "txt": txt.clone(), "t": timesteps.clone(), "y": y.clone() if y is not None else None,
                      "g": guidance.clone() if guidance is not None else None, "rope": rope,
                      "img_ids": img_ids, "txt_ids": txt_ids}
            run = lambda: self.forward(static["img"], static["img_ids"], static["txt"], static["txt_ids"],  # noqa: E731
                                       static["t"], static["y"], static["g"], rope=static["rope"])
            side = torch.cuda.Stream(device=img.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()                       # warm-up on the capture stream
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            if self.comm.world > 1:
                self.comm.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static["out"] = run()
            static["launches"] = self.launches
            g = st[key] = (graph, static)
        graph, static = g
        static["img"].copy_(img)
        static["txt"].copy_(txt)
        static["t"].copy_(timesteps)
        if y is not None:
            static["y"].copy_(y)
        if guidance is not None:
            static["g"].copy_(guidance)
        graph.replay()
        self.launches = static["launches"]
        return static["out"]

    # ---------------------------------------------------------------------------------------------------------
    # sequence parallel
    # ---------------------------------------------------------------------------------------------------------
    def _sp_context(self, S: int, St: int):
        from ..parallel.sp import UlyssesContext

        key = (S, St)
        if getattr(self, "_sp_key", None) != key:
            self._sp_ctx = UlyssesContext(self.comm, S, St, self.cfg.num_heads, self.cfg.hidden_size,
                                          self.cfg.mlp_hidden)
            self._sp_key = key
        return self._sp_ctx

    def _forward_sp(self, img, img_ids, txt, txt_ids, timesteps, y, guidance, rope):
        import os

        trace = os.environ.get("SWB_SP_TRACE") == "1" and not torch.cuda.is_current_stream_capturing()
        marks: list = []

        def mark(name):      # phase boundaries as CUDA events (profiling aid; eager mode only)
            if trace:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append((name, e))

        cfg, comm = self.cfg, self.comm
        H, D, NH, M = cfg.hidden_size, cfg.head_dim, cfg.num_heads, cfg.mlp_hidden
        P, r = comm.world, comm.rank
        B, Si, _ = img.shape
        assert B == 1, "sequence-parallel forward handles one image per call"
        St = txt.shape[1]
        S = St + Si
        dev = img.device
        self.launches = 0
        fused = os.environ.get("SWB_SP", "fused") != "nccl"
        if rope is None:
            rope = rope_table(torch.cat([txt_ids, img_ids], 0).to(dev), cfg.axes_dim, cfg.theta)
        cos, sin = rope
        St_l, Si_l = St // P, Si // P
        S_l, Hl = St_l + Si_l, NH // P
        scale = D ** -0.5
        sv = self.conditioning_vector(timesteps, y, guidance)
        mod = self._all_modulations(sv)
        x_txt = self._lin(txt[0, r * St_l:(r + 1) * St_l], "txt_in")          # [St_l, H]
        x_img = self._lin(img[0, r * Si_l:(r + 1) * Si_l], "img_in")          # [Si_l, H]
        positions = torch.arange(S, dtype=torch.int32, device=dev)
        # global positions of this rank's local rows ([txt_l | img_l])
        local_pos = torch.cat([positions[r * St_l:(r + 1) * St_l], positions[St + r * Si_l:St + (r + 1) * Si_l]])
        if fused:
            ctx = self._sp_context(S, St)
            buf2 = ctx.attn                                                     # [S_l, H + M], peers write [:, :H]
        else:
            buf2 = torch.empty((S_l, H + M), dtype=torch.bfloat16, device=dev)
            qkv_l = torch.empty((S_l, 3 * H), dtype=torch.bfloat16, device=dev)

        def exchange_and_attend(norms):
            """norms: [(row_lo, row_hi, q_norm, k_norm)] in GLOBAL rows (fused) or LOCAL rows (baseline)."""
            if fused:
                mark("qkv_gemm_scatter")
                ctx.barrier()                                   # every peer's QKV tiles have landed
                mark("barrier_a")
                for lo, hi, qn, kn in norms:
                    ops.rope_kv_write(ctx.qkv[lo:hi], positions[lo:hi], None, cos, sin, None, None, Hl, Hl, D,
                                      rot_dim=D, interleaved=True, q_norm=qn, k_norm=kn, norm_eps=1e-6)
                mark("rope")
                ctx.attn_scatter(scale)
                mark("attn_scatter")
                ctx.barrier()                                   # every peer's attention rows have landed
                mark("barrier_b")
                self.launches += 3 + len(norms)
                return
            for lo, hi, qn, kn in norms:
                ops.rope_kv_write(qkv_l[lo:hi], local_pos[lo:hi], None, cos, sin, None, None, NH, NH, D, rot_dim=D,
                                  interleaved=True, q_norm=qn, k_norm=kn, norm_eps=1e-6)
            g = comm.all_to_all(qkv_l.view(S_l, 3, NH, D), split_dim=2, cat_dim=0)       # [P*S_l, 3, Hl, D]
            o = ops.dense_attention(g[None, :, 0], g[None, :, 1], g[None, :, 2], scale=scale)[0]  # [P*S_l, Hl*D]
            back = comm.all_to_all(o.contiguous(), split_dim=0, cat_dim=1)               # [S_l, H]
            buf2[:, :H].copy_(back)
            self.launches += 2 + len(norms)

        mark("prologue")
        for i in range(cfg.depth):
            mods, norms = {}, []
            for s in ("img", "txt"):
                m = mod[f"double_blocks.{i}.{s}_mod.lin"]
                mods[s] = [m[:, j * H:(j + 1) * H] for j in range(6)]
            mark("rest")
            for s, x, lo_l, n_l, lo_g, n_g in (("txt", x_txt, 0, St_l, 0, St), ("img", x_img, St_l, Si_l, St, Si)):
                xm = ops.layernorm_mod(x[None], scale=mods[s][1], shift=mods[s][0], rows_per_batch=n_l)[0]
                name = f"double_blocks.{i}.{s}_attn.qkv"
                if fused:
                    ctx.gemm_scatter(xm, self.w[name + ".weight"], self.w[name + ".bias"], s)
                    self.launches += 1
                else:
                    self._lin(xm, name, out=qkv_l[lo_l:lo_l + n_l])
                nw = (self.w[f"double_blocks.{i}.{s}_attn.norm.query_norm.scale"],
                      self.w[f"double_blocks.{i}.{s}_attn.norm.key_norm.scale"])
                norms.append((lo_g, lo_g + n_g, *nw) if fused else (lo_l, lo_l + n_l, *nw))
            exchange_and_attend(norms)
            new = {}
            for s, x, lo_l, n_l in (("txt", x_txt, 0, St_l), ("img", x_img, St_l, Si_l)):
                proj = self._lin(buf2[lo_l:lo_l + n_l, :H], f"double_blocks.{i}.{s}_attn.proj")
                x = ops.gated_residual(x[None], proj[None], mods[s][2], rows_per_batch=n_l)
                hm = ops.layernorm_mod(x, scale=mods[s][4], shift=mods[s][3], rows_per_batch=n_l)
                h1 = self._lin(hm[0], f"double_blocks.{i}.{s}_mlp.0", act="gelu_tanh")
                h2 = self._lin(h1, f"double_blocks.{i}.{s}_mlp.2")
                new[s] = ops.gated_residual(x, h2[None], mods[s][5], rows_per_batch=n_l)[0]
                self.launches += 3
            x_img, x_txt = new["img"], new["txt"]

        x = torch.cat([x_txt, x_img], 0).contiguous()                           # [S_l, H] local joint
        for i in range(cfg.depth_single):
            p = f"single_blocks.{i}"
            m = mod[p + ".modulation.lin"]
            sh, sc, g = m[:, :H], m[:, H:2 * H], m[:, 2 * H:]
            mark("rest")
            xm = ops.layernorm_mod(x[None], scale=sc, shift=sh, rows_per_batch=S_l)[0]
            nw = (self.w[p + ".norm.query_norm.scale"], self.w[p + ".norm.key_norm.scale"])
            if fused:
                ctx.gemm_scatter(xm, self.w[p + ".linear1_qkv.weight"], self.w[p + ".linear1_qkv.bias"], "joint")
                self.launches += 1
            else:
                self._lin(xm, p + ".linear1_qkv", out=qkv_l)
            self._lin(xm, p + ".linear1_mlp", act="gelu_tanh", out=buf2[:, H:])
            exchange_and_attend([(0, S, *nw)] if fused else [(0, S_l, *nw)])
            out = self._lin(buf2, p + ".linear2")
            x = ops.gated_residual(x[None], out[None], g, rows_per_batch=S_l)[0]
            self.launches += 2
        x_img = x[St_l:].contiguous()
        m = mod["final_layer.adaLN_modulation.1"]
        xm = ops.layernorm_mod(x_img[None], scale=m[:, H:], shift=m[:, :H], rows_per_batch=Si_l)[0]
        v_local = self._lin(xm, "final_layer.linear")                           # [Si_l, C]
        self.launches += 2
        out = comm.all_gather(v_local, dim=0)[None]
        if trace:
            mark("rest")
            torch.cuda.synchronize()
            tot: dict = {}
            for (_, e0), (name, e1) in zip(marks, marks[1:]):
                tot[name] = tot.get(name, 0.0) + e0.elapsed_time(e1)
            self.sp_phase_ms = {k: round(v, 3) for k, v in tot.items()}
        return out
