"""Qwen3.5 / Qwen3-Next hybrid decoder: three Gated-DeltaNet (linear attention) layers for every gated full-attention
layer, partial rotary embedding, (1 + w) RMSNorm (candle-llm/src/primitives/gated_delta.rs:1-432,
candle-llm/src/models/qwen35.rs:1-1674).

Gated DeltaNet keeps, per value head, a [d_k, d_v] state S updated token by token:
    S <- exp(g_t) * S;   S <- S + k_t (x) (beta_t * (v_t - S^T k_t));   o_t = S^T (q_t / sqrt(d_k))
with q, k L2-normalised, g_t = -exp(A_log) * softplus(a_t + dt_bias) and beta_t = sigmoid(b_t). q, k, v first pass a
causal depthwise convolution (kernel 4) + SiLU whose last 3 inputs are the second piece of per-layer state. The output is
RMS-normalised per head and gated by SiLU(z).

The class exposes the oracle decoder surface (`make_cache`, `decode_logits`, `decode_logits_all`, `generate_greedy`),
so the decode loops and the provider host it like any other model. Projections run on the tcgen05 GEMM for bf16
weights on a CUDA device; the recurrence is a sequential fp32 scan (state tensors [B, H, d_k, d_v])."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from ..contracts.errors import ConfigError, LoadError, Unsupported
from .text_encoders import linear


# ---- Gated DeltaNet primitives -------------------------------------------------------------------------------------------
def compute_g(a: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor) -> torch.Tensor:
    """Log decay per token and head: -exp(A_log) * softplus(a + dt_bias), fp32."""
    return -a_log.float().exp() * F.softplus(a.float() + dt_bias.float())


def causal_depthwise_conv(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None
                          ) -> tuple[torch.Tensor, torch.Tensor]:
    """x [B, T, C], weight [C, K], state [B, K - 1, C] (the inputs before this call; zeros at the start).
    Returns (SiLU(conv(x)) [B, T, C], new state = the last K - 1 inputs)."""
    B, T, C = x.shape
    K = weight.shape[1]
    if state is None:
        state = torch.zeros(B, K - 1, C, dtype=x.dtype, device=x.device)
    full = torch.cat([state, x], dim=1)                                   # [B, K - 1 + T, C]
    y = F.conv1d(full.transpose(1, 2).float(), weight.float().unsqueeze(1), groups=C).transpose(1, 2)
    return F.silu(y).to(x.dtype), full[:, -(K - 1):].contiguous()


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta_recurrence(q, k, v, g, beta, state: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
    """q, k [B, T, H, d_k]; v [B, T, H, d_v]; g, beta [B, T, H]; state [B, H, d_k, d_v] or None.
    Returns (o [B, T, H, d_v], final state), all fp32."""
    q, k, v, g, beta = (t.float() for t in (q, k, v, g, beta))
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    q = l2norm(q) * dk ** -0.5
    k = l2norm(k)
    S = torch.zeros(B, H, dk, dv, device=q.device) if state is None else state.float().clone()
    out = torch.empty(B, T, H, dv, device=q.device)
    for t in range(T):
        S = S * g[:, t].exp()[..., None, None]
        kt = k[:, t]
        delta = (v[:, t] - torch.einsum("bhkv,bhk->bhv", S, kt)) * beta[:, t][..., None]
        S = S + kt[..., None] * delta[..., None, :]
        out[:, t] = torch.einsum("bhkv,bhk->bhv", S, q[:, t])
    return out, S


def rms_norm_gated(x: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * rmsnorm(x) * SiLU(gate): normalised first, then gated."""
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.float() * xf * F.silu(gate.float())).to(x.dtype)


# ---- configuration -----------------------------------------------------------------------------------------------------
@dataclass
class Qwen35Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    linear_num_value_heads: int
    linear_num_key_heads: int
    linear_key_head_dim: int
    linear_value_head_dim: int
    linear_conv_kernel_dim: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10_000_000.0
    partial_rotary_factor: float = 0.25
    full_attention_interval: int = 4
    layer_types: list[str] = field(default_factory=list)
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 0

    @classmethod
    def from_json(cls, top: dict) -> "Qwen35Config":
        v = top.get("text_config", top)
        try:
            rp = v.get("rope_parameters") or v.get("rope_scaling") or {}
            cfg = cls(
                vocab_size=int(v["vocab_size"]), hidden_size=int(v["hidden_size"]),
                intermediate_size=int(v["intermediate_size"]), num_hidden_layers=int(v["num_hidden_layers"]),
                num_attention_heads=int(v["num_attention_heads"]), num_key_value_heads=int(v["num_key_value_heads"]),
                head_dim=int(v.get("head_dim") or v["hidden_size"] // v["num_attention_heads"]),
                linear_num_value_heads=int(v["linear_num_value_heads"]),
                linear_num_key_heads=int(v["linear_num_key_heads"]), linear_key_head_dim=int(v["linear_key_head_dim"]),
                linear_value_head_dim=int(v["linear_value_head_dim"]),
                linear_conv_kernel_dim=int(v.get("linear_conv_kernel_dim", 4)),
                rms_norm_eps=float(v.get("rms_norm_eps", 1e-6)),
                rope_theta=float(rp.get("rope_theta", v.get("rope_theta", 10_000_000.0))),
                partial_rotary_factor=float(rp.get("partial_rotary_factor", v.get("partial_rotary_factor", 0.25))),
                full_attention_interval=int(v.get("full_attention_interval", 4)),
                layer_types=list(v.get("layer_types") or []),
                tie_word_embeddings=bool(top.get("tie_word_embeddings", v.get("tie_word_embeddings", False))),
                max_position_embeddings=int(v.get("max_position_embeddings", 0)))
        except KeyError as e:
            raise ConfigError(f"qwen3.5 config.json missing `{e.args[0]}`") from e
        if not cfg.layer_types:
            n = cfg.full_attention_interval
            cfg.layer_types = ["full_attention" if (i + 1) % n == 0 else "linear_attention"
                               for i in range(cfg.num_hidden_layers)]
        return cfg

    def is_linear(self, i: int) -> bool:
        return self.layer_types[i] == "linear_attention"

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def num_layers(self) -> int:
        return self.num_hidden_layers


# ---- cache ---------------------------------------------------------------------------------------------------------------
class Qwen35Cache:
    """Per layer either (K, V) of a full-attention layer or (conv state, recurrent state) of a DeltaNet layer."""

    def __init__(self, cfg: Qwen35Config):
        self.cfg = cfg
        self.kv: list[tuple[torch.Tensor, torch.Tensor] | None] = [None] * cfg.num_hidden_layers
        self.lin: list[tuple[torch.Tensor, torch.Tensor] | None] = [None] * cfg.num_hidden_layers
        self._offset = 0

    @property
    def offset(self) -> int:
        return self._offset

    def reset(self) -> None:
        self.kv = [None] * self.cfg.num_hidden_layers
        self.lin = [None] * self.cfg.num_hidden_layers
        self._offset = 0

    def truncate(self, length: int) -> None:
        """A recurrent state cannot be rolled back: only a no-op or a full reset is possible."""
        if length == self._offset:
            return
        if length == 0:
            self.reset()
            return
        raise Unsupported("a Gated-DeltaNet state cannot be truncated to an earlier position")

    def clone(self) -> "Qwen35Cache":
        c = Qwen35Cache(self.cfg)
        c.kv = [None if e is None else (e[0].clone(), e[1].clone()) for e in self.kv]
        c.lin = [None if e is None else (e[0].clone(), e[1].clone()) for e in self.lin]
        c._offset = self._offset
        return c


# ---- model ---------------------------------------------------------------------------------------------------------------
class Qwen35Model:
    def __init__(self, cfg: Qwen35Config, weights: dict[str, torch.Tensor], dtype: torch.dtype = torch.float32,
                 device: str | torch.device = "cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        w = {}
        for k, v in weights.items():
            k = k.replace("model.language_model.", "model.")
            if k.startswith(("model.embed_tokens", "model.layers.", "model.norm", "lm_head")):
                w[k] = v.to(self.device, dtype if v.is_floating_point() else v.dtype)
        if "model.embed_tokens.weight" not in w:
            raise LoadError("missing model.embed_tokens.weight")
        if "lm_head.weight" not in w:
            w["lm_head.weight"] = w["model.embed_tokens.weight"]
        self.w = w
        rd = cfg.rotary_dim
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float32, device=self.device) / rd))

    def make_cache(self) -> Qwen35Cache:
        return Qwen35Cache(self.cfg)

    def _norm(self, x: torch.Tensor, key: str) -> torch.Tensor:
        xf = x.float()
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)
        return (xf * (1.0 + self.w[key].float())).to(x.dtype)

    def _lin(self, x: torch.Tensor, key: str) -> torch.Tensor:
        return linear(x, self.w[key + ".weight"], self.w.get(key + ".bias"))

    def _rope(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x [B, H, T, D]: rotate the first rotary_dim features (half-split pairs), pass the rest through."""
        rd = self.cfg.rotary_dim
        xr, xp = x[..., :rd].float(), x[..., rd:]
        x1, x2 = xr[..., : rd // 2], xr[..., rd // 2:]
        rot = torch.cat([-x2, x1], dim=-1)
        return torch.cat([(xr * cos + rot * sin).to(x.dtype), xp], dim=-1)

    def _full_attention(self, h, i, cos, sin, cache: Qwen35Cache | None) -> torch.Tensor:
        c = self.cfg
        p = f"model.layers.{i}.self_attn"
        B, T, _ = h.shape
        Hq, Hkv, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        qg = self._lin(h, p + ".q_proj").view(B, T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(B, T, Hq * D)
        q = self._norm(q, p + ".q_norm.weight").transpose(1, 2)
        k = self._norm(self._lin(h, p + ".k_proj").view(B, T, Hkv, D), p + ".k_norm.weight").transpose(1, 2)
        v = self._lin(h, p + ".v_proj").view(B, T, Hkv, D).transpose(1, 2)
        q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
        if cache is not None:
            if cache.kv[i] is not None:
                k, v = torch.cat([cache.kv[i][0], k], dim=2), torch.cat([cache.kv[i][1], v], dim=2)
            cache.kv[i] = (k, v)
        S = k.shape[2]
        rep = Hq // Hkv
        kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        mask = torch.ones(T, S, dtype=torch.bool, device=h.device).tril(diagonal=S - T)
        a = F.scaled_dot_product_attention(q.float(), kk.float(), vv.float(), attn_mask=mask, scale=D ** -0.5)
        a = a.transpose(1, 2).reshape(B, T, Hq * D).to(h.dtype)
        return self._lin(a * torch.sigmoid(gate.float()).to(h.dtype), p + ".o_proj")

    def _delta_net(self, h, i, cache: Qwen35Cache | None) -> torch.Tensor:
        c = self.cfg
        p = f"model.layers.{i}.linear_attn"
        B, T, _ = h.shape
        Hv, Hk, dk, dv = c.linear_num_value_heads, c.linear_num_key_heads, c.linear_key_head_dim, c.linear_value_head_dim
        key_dim = Hk * dk
        qkv = self._lin(h, p + ".in_proj_qkv")
        z = self._lin(h, p + ".in_proj_z").view(B, T, Hv, dv)
        b, a = self._lin(h, p + ".in_proj_b"), self._lin(h, p + ".in_proj_a")
        conv_state, ssm_state = cache.lin[i] if cache is not None and cache.lin[i] is not None else (None, None)
        qkv, conv_state = causal_depthwise_conv(qkv, self.w[p + ".conv1d.weight"].squeeze(1), conv_state)
        q, k, v = qkv[..., :key_dim], qkv[..., key_dim:2 * key_dim], qkv[..., 2 * key_dim:]
        q, k, v = q.reshape(B, T, Hk, dk), k.reshape(B, T, Hk, dk), v.reshape(B, T, Hv, dv)
        if Hv // Hk > 1:
            q, k = q.repeat_interleave(Hv // Hk, dim=2), k.repeat_interleave(Hv // Hk, dim=2)
        g = compute_g(a, self.w[p + ".A_log"], self.w[p + ".dt_bias"])
        o, ssm_state = gated_delta_recurrence(q, k, v, g, torch.sigmoid(b.float()), ssm_state)
        if cache is not None:
            cache.lin[i] = (conv_state, ssm_state)
        o = rms_norm_gated(o.to(h.dtype), self.w[p + ".norm.weight"], z, c.rms_norm_eps).reshape(B, T, Hv * dv)
        return self._lin(o, p + ".out_proj")

    @torch.no_grad()
    def hidden_states(self, ids: torch.Tensor | None, cache: Qwen35Cache | None, offset: int = 0, *,
                      embeds: torch.Tensor | None = None) -> torch.Tensor:
        x = self.w["model.embed_tokens.weight"][ids.to(self.device)] if embeds is None else embeds.to(self.device,
                                                                                                       self.dtype)
        B, T, _ = x.shape
        pos = torch.arange(offset, offset + T, device=self.device, dtype=torch.float32)
        fr = pos[:, None] * self.inv_freq[None, :]
        emb = torch.cat([fr, fr], dim=-1)
        cos, sin = emb.cos()[None, None], emb.sin()[None, None]
        for i in range(self.cfg.num_hidden_layers):
            p = f"model.layers.{i}"
            h = self._norm(x, p + ".input_layernorm.weight")
            x = x + (self._delta_net(h, i, cache) if self.cfg.is_linear(i) else self._full_attention(h, i, cos, sin, cache))
            h = self._norm(x, p + ".post_attention_layernorm.weight")
            gate, up = self._lin(h, p + ".mlp.gate_proj"), self._lin(h, p + ".mlp.up_proj")
            x = x + self._lin((F.silu(gate.float()) * up.float()).to(x.dtype), p + ".mlp.down_proj")
        if cache is not None:
            cache._offset = offset + T
        return x

    def project_logits(self, h: torch.Tensor) -> torch.Tensor:
        return self._norm(h, "model.norm.weight").float() @ self.w["lm_head.weight"].float().t()

    @torch.no_grad()
    def decode_logits(self, ids: torch.Tensor, cache: Qwen35Cache | None, offset: int = 0, **kw) -> torch.Tensor:
        return self.project_logits(self.hidden_states(ids, cache, offset, **kw)[:, -1:, :])[:, 0]

    @torch.no_grad()
    def decode_logits_all(self, ids: torch.Tensor, cache: Qwen35Cache | None, offset: int = 0, **kw) -> torch.Tensor:
        return self.project_logits(self.hidden_states(ids, cache, offset, **kw))

    @torch.no_grad()
    def generate_greedy(self, prompt: list[int], max_new_tokens: int, stop_tokens: tuple[int, ...] = ()
                        ) -> tuple[list[int], list[float]]:
        cache = self.make_cache()
        logits = self.decode_logits(torch.tensor([prompt], dtype=torch.long), cache, 0)
        out, margins = [], []
        for _ in range(max_new_tokens):
            top2 = logits[0].float().topk(2).values
            margins.append(float(top2[0] - top2[1]))
            tok = int(torch.argmax(logits[0].float()))
            if tok in stop_tokens:
                break
            out.append(tok)
            logits = self.decode_logits(torch.tensor([[tok]], dtype=torch.long), cache, cache.offset)
        return out, margins
