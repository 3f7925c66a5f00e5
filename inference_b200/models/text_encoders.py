"""T5 (v1.1, encoder only) and CLIP text encoders: the two prompt encoders of FLUX-family pipelines
(candle-gen-flux/src/pipeline.rs:552-620 encodes with T5-XXL [1, L, 4096] and takes CLIP-L's pooled vector [1, 768]).

Both are written once over torch tensors; `linear` routes every projection through the tcgen05 GEMM when the weights
are bf16 on a CUDA device and through a plain matmul otherwise (CPU oracle backend). Attention runs on small
[heads, L, L] score tensors (L <= 512, head dim 64) and stays in torch. Weight names follow the Hugging Face
checkpoints (`encoder.block.N.layer.0.SelfAttention.q.weight`, `text_model.encoder.layers.N.self_attn.q_proj.weight`)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    if x.is_cuda and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0:
        from .. import ops

        lead = x.shape[:-1]
        y = ops.gemm_bf16(x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous(), w, bias=b)
        return y.reshape(*lead, w.shape[0])
    y = x.to(w.dtype) @ w.t()
    return y + b if b is not None else y


# ---------------------------------------------------------------------------------------------------------------
# T5 encoder
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 4096
    d_kv: int = 64
    d_ff: int = 10240
    num_layers: int = 24
    num_heads: int = 64
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6

    @staticmethod
    def from_json(j: dict) -> "T5Config":
        keys = T5Config.__dataclass_fields__
        return T5Config(**{k: j[k] for k in keys if k in j})


def _t5_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional bucketing of relative positions (memory - query)."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    n = rel.abs()
    max_exact = nb // 2
    large = max_exact + (torch.log(n.float().clamp_min(1) / max_exact) / math.log(max_distance / max_exact)
                         * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return out + torch.where(n < max_exact, n, large)


class T5Encoder:
    def __init__(self, cfg: T5Config, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()
                  if k.startswith(("encoder.", "shared."))}
        if "shared.weight" not in self.w and "encoder.embed_tokens.weight" in self.w:
            self.w["shared.weight"] = self.w["encoder.embed_tokens.weight"]

    def _norm(self, x, name):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(v + self.cfg.layer_norm_epsilon)).to(self.dtype) * self.w[name]

    @torch.no_grad()
    def encode(self, ids: torch.Tensor, mask: torch.Tensor | None = None) -> torch.Tensor:
        """ids [B, L] int64 -> last hidden state [B, L, d_model]. `mask` [B, L] (1 = attend); FLUX passes none and
        attends the padding too."""
        cfg = self.cfg
        B, L = ids.shape
        H, D = cfg.num_heads, cfg.d_kv
        x = self.w["shared.weight"][ids.to(self.device)]
        pos = torch.arange(L, device=self.device)
        buckets = _t5_bucket(pos[None, :] - pos[:, None], cfg.relative_attention_num_buckets,
                             cfg.relative_attention_max_distance)
        neg = None
        if mask is not None:
            neg = (1.0 - mask.to(self.device).float())[:, None, None, :] * torch.finfo(torch.float32).min
        bias = None
        for i in range(cfg.num_layers):
            p = f"encoder.block.{i}.layer"
            # T5 shares the first layer's relative-position table; UMT5 stores one per layer
            table = self.w.get(f"{p}.0.SelfAttention.relative_attention_bias.weight")                 # [buckets, H]
            if table is not None:
                bias = table[buckets].permute(2, 0, 1)[None].float()                                  # [1, H, L, L]
                if neg is not None:
                    bias = bias + neg
            h = self._norm(x, f"{p}.0.layer_norm.weight")
            q, k, v = (linear(h, self.w[f"{p}.0.SelfAttention.{n}.weight"]).view(B, L, H, D).transpose(1, 2)
                       for n in "qkv")
            s = q.float() @ k.float().transpose(-1, -2) + bias          # T5 does not scale by sqrt(d)
            a = (torch.softmax(s, -1) @ v.float()).transpose(1, 2).reshape(B, L, H * D).to(self.dtype)
            x = x + linear(a, self.w[f"{p}.0.SelfAttention.o.weight"])
            h = self._norm(x, f"{p}.1.layer_norm.weight")
            g = F.gelu(linear(h, self.w[f"{p}.1.DenseReluDense.wi_0.weight"]).float(), approximate="tanh")
            u = linear(h, self.w[f"{p}.1.DenseReluDense.wi_1.weight"]).float()
            x = x + linear((g * u).to(self.dtype), self.w[f"{p}.1.DenseReluDense.wo.weight"])
        return self._norm(x, "encoder.final_layer_norm.weight")


# ---------------------------------------------------------------------------------------------------------------
# CLIP text encoder
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class ClipTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 77
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"
    eos_token_id: int = 49407

    @staticmethod
    def from_json(j: dict) -> "ClipTextConfig":
        j = j.get("text_config", j)
        keys = ClipTextConfig.__dataclass_fields__
        return ClipTextConfig(**{k: j[k] for k in keys if k in j})


class ClipTextEncoder:
    def __init__(self, cfg: ClipTextConfig, weights: dict[str, torch.Tensor], device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(device=self.device, dtype=dtype).contiguous() for k, v in weights.items()
                  if k.startswith(("text_model.", "text_projection."))}

    def _ln(self, x, name):
        return F.layer_norm(x.float(), (x.shape[-1],), self.w[name + ".weight"].float(), self.w[name + ".bias"].float(),
                            self.cfg.layer_norm_eps).to(self.dtype)

    def _act(self, x):
        x = x.float()
        if self.cfg.hidden_act == "quick_gelu":
            return x * torch.sigmoid(1.702 * x)
        return F.gelu(x)

    @torch.no_grad()
    def encode(self, ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """ids [B, L <= 77] -> (last hidden state [B, L, hidden], pooled [B, hidden] = state at the first EOS token)."""
        out = self.encode_all(ids)
        return out["last"], out["pooled"]

    @torch.no_grad()
    def encode_all(self, ids: torch.Tensor) -> dict[str, torch.Tensor]:
        """last / pooled as in encode(), `penultimate` = the input of the final layer (Hugging Face
        `hidden_states[-2]`, no final LayerNorm) and, when the checkpoint has a `text_projection`, `projected` = the
        pooled vector through it (`text_embeds`)."""
        cfg = self.cfg
        B, L = ids.shape
        H = cfg.num_attention_heads
        D = cfg.hidden_size // H
        ids = ids.to(self.device)
        p = "text_model."
        x = self.w[p + "embeddings.token_embedding.weight"][ids] + self.w[p + "embeddings.position_embedding.weight"][:L]
        causal = torch.full((L, L), float("-inf"), device=self.device).triu(1)
        penultimate = x
        for i in range(cfg.num_hidden_layers):
            lp = f"{p}encoder.layers.{i}."
            if i == cfg.num_hidden_layers - 1:
                penultimate = x
            h = self._ln(x, lp + "layer_norm1")
            q, k, v = (linear(h, self.w[f"{lp}self_attn.{n}_proj.weight"], self.w[f"{lp}self_attn.{n}_proj.bias"])
                       .view(B, L, H, D).transpose(1, 2).float() for n in "qkv")
            s = q @ k.transpose(-1, -2) * D ** -0.5 + causal
            a = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, L, H * D).to(self.dtype)
            x = x + linear(a, self.w[lp + "self_attn.out_proj.weight"], self.w[lp + "self_attn.out_proj.bias"])
            h = self._ln(x, lp + "layer_norm2")
            h = self._act(linear(h, self.w[lp + "mlp.fc1.weight"], self.w[lp + "mlp.fc1.bias"])).to(self.dtype)
            x = x + linear(h, self.w[lp + "mlp.fc2.weight"], self.w[lp + "mlp.fc2.bias"])
        x = self._ln(x, p + "final_layer_norm")
        if cfg.eos_token_id == 2:                     # legacy checkpoints: the EOS has the largest id
            eos = ids.argmax(-1)
        else:
            eos = (ids == cfg.eos_token_id).int().argmax(-1)
        pooled = x[torch.arange(B, device=self.device), eos]
        out = {"last": x, "pooled": pooled, "penultimate": penultimate}
        if "text_projection.weight" in self.w:
            out["projected"] = linear(pooled, self.w["text_projection.weight"])
        return out


# ---------------------------------------------------------------------------------------------------------------
# decoder-only language model used as a prompt encoder
# ---------------------------------------------------------------------------------------------------------------
class CausalLmTextEncoder:
    """Hidden states of a Llama-family decoder after all but `skip_last` of its layers, before the final norm
    (Z-Image and its relatives condition on the second-to-last layer of Qwen3: candle-gen-z-image/src/pipeline.rs:115-127).

    On a CUDA device with head_dim 128 the stack runs on the sm_100a kernels (one fused q/k/v GEMM, q/k RMSNorm + RoPE
    in place, causal tcgen05 attention, gated-pair MLP GEMM); elsewhere it is the fp32 oracle decoder."""

    def __init__(self, cfg, weights: dict[str, torch.Tensor], device="cpu", skip_last: int = 1, final_norm: bool = False):
        from .oracle import OracleLlama, canonical_weights
        from .config import build_rope

        self.cfg, self.device = cfg, torch.device(device)
        self.layers = cfg.num_layers - skip_last
        self.final_norm = final_norm            # Qwen-Image conditions on the last layer after the model's final norm
        self.native = (self.device.type == "cuda" and cfg.head_dim == 128 and not cfg.is_moe and cfg.mla is None and
                       cfg.architecture.value in ("llama", "qwen3"))
        if not self.native:
            self.oracle = OracleLlama(cfg, weights, torch.float32, self.device)
            return
        w = canonical_weights(weights, cfg)
        dev = self.device
        bf = lambda t: t.to(device=dev, dtype=torch.bfloat16).contiguous()      # noqa: E731
        self.embed = bf(w["model.embed_tokens.weight"])
        self.norm_w = bf(w["model.norm.weight"]) if final_norm else None
        self.blocks = []
        for i in range(self.layers):
            p = f"model.layers.{i}."
            qkv = torch.cat([w[p + f"self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0)
            bias = None
            if p + "self_attn.q_proj.bias" in w:
                bias = bf(torch.cat([w[p + f"self_attn.{n}_proj.bias"] for n in ("q", "k", "v")], 0))
            gate, up = w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]
            self.blocks.append({
                "ln1": bf(w[p + "input_layernorm.weight"]), "ln2": bf(w[p + "post_attention_layernorm.weight"]),
                "qkv": bf(qkv), "qkv_bias": bias, "o": bf(w[p + "self_attn.o_proj.weight"]),
                "q_norm": bf(w[p + "self_attn.q_norm.weight"]) if p + "self_attn.q_norm.weight" in w else None,
                "k_norm": bf(w[p + "self_attn.k_norm.weight"]) if p + "self_attn.k_norm.weight" in w else None,
                "gate_up": bf(torch.stack([gate, up], 1).reshape(-1, gate.shape[1])), "down": bf(w[p + "mlp.down_proj.weight"])})
        rope = build_rope(cfg)
        self.inv_freq = torch.tensor(rope.inv_freq, dtype=torch.float32, device=dev)
        self.rot_dim, self.rope_interleaved = rope.dim, rope.interleaved

    @torch.no_grad()
    def encode_layers(self, ids: list[int], select: list[int]) -> torch.Tensor:
        """token ids -> [1, len(ids), len(select), hidden]: the residual stream after `select[j]` decoder layers
        (0 = the embeddings), stacked along a new axis (Krea conditions on twelve layers of its encoder:
        candle-gen-krea/src/text_encoder.rs:41-56,491-520). Needs skip_last small enough to reach max(select)."""
        if max(select) > self.layers:
            raise ValueError(f"layer {max(select)} requested but the encoder keeps {self.layers} layers")
        if not self.native:
            t = torch.tensor([ids], dtype=torch.int64, device=self.device)
            return torch.stack([self.oracle.hidden_states(t, None, num_layers=i) for i in select], dim=2)
        taps: dict[int, torch.Tensor] = {}
        self.encode(ids, _taps=(set(select), taps))
        return torch.stack([taps[i] for i in select], dim=1)[None]

    @torch.no_grad()
    def encode(self, ids: list[int], _taps=None) -> torch.Tensor:
        """token ids -> [1, len(ids), hidden]."""
        t = torch.tensor([ids], dtype=torch.int64, device=self.device)
        if not self.native:
            h = self.oracle.hidden_states(t, None, num_layers=self.layers)
            return self.oracle._norm(h, "model.norm.weight") if self.final_norm else h
        from .. import ops

        cfg = self.cfg
        S, D, Hq, Hkv = len(ids), cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        eps, woff = cfg.rms_norm_eps, cfg.norm_weight_offset
        pos = torch.arange(S, dtype=torch.int32, device=self.device)
        ang = pos.float()[:, None] * self.inv_freq[None]
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        x = ops.embedding(t, self.embed, scale=cfg.embed_scale)
        if _taps is not None and 0 in _taps[0]:
            _taps[1][0] = x.clone()
        for li, b in enumerate(self.blocks):
            if _taps is not None and li > 0 and li in _taps[0]:
                _taps[1][li] = x.clone()
            qkv = ops.gemm_bf16(ops.rmsnorm(x, b["ln1"], eps, w_offset=woff), b["qkv"], bias=b["qkv_bias"])
            ops.rope_kv_write(qkv, pos, None, cos, sin, None, None, Hq, Hkv, D, rot_dim=self.rot_dim,
                              interleaved=self.rope_interleaved, q_norm=b["q_norm"], k_norm=b["k_norm"], norm_eps=eps,
                              norm_w_offset=woff)
            q3 = qkv.view(1, S, Hq + 2 * Hkv, D)
            attn = ops.dense_attention(q3[:, :, :Hq], q3[:, :, Hq:Hq + Hkv], q3[:, :, Hq + Hkv:], scale=cfg.attn_scale,
                                       causal=True)
            x = ops.gemm_bf16(attn.view(S, Hq * D), b["o"], residual=x)
            h = ops.linear_gated(ops.rmsnorm(x, b["ln2"], eps, w_offset=woff), b["gate_up"],
                                 cfg.mlp_activation)
            x = ops.gemm_bf16(h, b["down"], residual=x)
        if _taps is not None and len(self.blocks) in _taps[0]:
            _taps[1][len(self.blocks)] = x.clone()
        if self.final_norm:
            x = ops.rmsnorm(x, self.norm_w, eps, w_offset=woff)
        return x[None]
