"""fp32 PyTorch restatement of the reference decoder math: the correctness oracle and the CPU runtime.

Runs anywhere (CPU or a single CUDA device, any dtype) with plain PyTorch ops and a contiguous KV
cache. Every GPU kernel and the paged engine are tested against this model. Semantics restated from
candle-llm: linear `x @ W^T + b` (primitives/nn.rs:14-19), RMSNorm with fp32 statistics (nn.rs:21-32),
RoPE half-split / interleaved / partial (primitives/rope.rs), GQA via repeat_kv and
`softmax(scale * Q K^T + mask) V` with a bottom-right aligned causal mask of -1e30
(primitives/attention.rs:42-191), SwiGLU / GeGLU MLP (models/llama.rs:1378-1392), the Gemma-2 / GLM-4
four-norm sandwich (models/llama.rs:898-976), the top-k routed MoE FFN with shared expert
(models/llama.rs:1400-1488), final norm + (tied) lm_head + optional logit soft-cap (models/llama.rs:714-725).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..contracts.errors import LoadError
from .config import Architecture, ModelConfig, build_rope

MASK_NEG = -1e30


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + offset)
    return y.to(x.dtype)


def rope_cos_sin(inv_freq: torch.Tensor, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    ang = positions.float()[..., None] * inv_freq.float()
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot_dim: int, interleaved: bool) -> torch.Tensor:
    """x [..., S, H, D]; cos/sin [..., S, rot_dim/2] broadcast over heads."""
    c, s = cos.unsqueeze(-2).to(x.dtype), sin.unsqueeze(-2).to(x.dtype)
    xr, xp = x[..., :rot_dim], x[..., rot_dim:]
    if interleaved:
        x0, x1 = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1).flatten(-2)
    else:
        h = rot_dim // 2
        x0, x1 = xr[..., :h], xr[..., h:]
        out = torch.cat((x0 * c - x1 * s, x1 * c + x0 * s), dim=-1)
    return torch.cat((out, xp), dim=-1) if xp.shape[-1] else out


def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, causal: bool,
         additive_mask: torch.Tensor | None = None, softcap: float | None = None) -> torch.Tensor:
    """q [B, Hq, Sq, D], k/v [B, Hkv, Sk, D] -> [B, Hq, Sq, D]; GQA by expanding k/v."""
    g = q.shape[1] // k.shape[1]
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if softcap:
        s = torch.tanh(s / softcap) * softcap
    sq, sk = q.shape[2], k.shape[2]
    if causal and sq > 1:
        i = torch.arange(sq, device=q.device)[:, None]
        j = torch.arange(sk, device=q.device)[None, :]
        s = s.masked_fill(j > i + (sk - sq), MASK_NEG)
    if additive_mask is not None:
        s = s + additive_mask.to(s.dtype)
    p = torch.softmax(s.float(), dim=-1).to(q.dtype)
    return torch.matmul(p, v)


@dataclass
class ContiguousKvCache:
    """Concat-grow per-layer K/V ([B, Hkv, S, D]); supports truncate for speculative rollback and row
    retention for batch compaction (candle-llm/src/primitives/kv_cache.rs:17-178)."""
    num_layers: int
    k: list[torch.Tensor | None] = field(default_factory=list)
    v: list[torch.Tensor | None] = field(default_factory=list)

    def __post_init__(self):
        self.k = [None] * self.num_layers
        self.v = [None] * self.num_layers

    @property
    def offset(self) -> int:
        return 0 if self.k[0] is None else self.k[0].shape[2]

    @property
    def batch_size(self) -> int:
        return 0 if self.k[0] is None else self.k[0].shape[0]

    def update(self, layer: int, k: torch.Tensor, v: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        if self.k[layer] is None:
            self.k[layer], self.v[layer] = k, v
        else:
            self.k[layer] = torch.cat((self.k[layer], k), dim=2)
            self.v[layer] = torch.cat((self.v[layer], v), dim=2)
        return self.k[layer], self.v[layer]

    def truncate(self, length: int) -> None:
        for i in range(self.num_layers):
            if self.k[i] is not None:
                self.k[i] = self.k[i][:, :, :length]
                self.v[i] = self.v[i][:, :, :length]

    def retain_sequences(self, rows: list[int]) -> None:
        idx = torch.tensor(rows, dtype=torch.long)
        for i in range(self.num_layers):
            if self.k[i] is not None:
                self.k[i] = self.k[i][idx.to(self.k[i].device)]
                self.v[i] = self.v[i][idx.to(self.v[i].device)]

    def reset(self) -> None:
        self.k = [None] * self.num_layers
        self.v = [None] * self.num_layers

    def clone(self) -> "ContiguousKvCache":
        c = ContiguousKvCache(self.num_layers)
        c.k = [None if t is None else t.clone() for t in self.k]
        c.v = [None if t is None else t.clone() for t in self.v]
        return c


def _split_packed(weights: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    """Phi-3 / GLM-4 packed qkv_proj and gate_up_proj -> standard projections (models/llama.rs:74-319)."""
    out = dict(weights)
    q_out = cfg.num_heads * cfg.head_dim
    kv_out = cfg.num_kv_heads * cfg.head_dim
    for key in list(weights):
        if key.endswith("self_attn.qkv_proj.weight") or key.endswith("self_attn.qkv_proj.bias"):
            base, kind = key.rsplit("qkv_proj.", 1)
            t = out.pop(key)
            out[f"{base}q_proj.{kind}"], out[f"{base}k_proj.{kind}"], out[f"{base}v_proj.{kind}"] = (
                t[:q_out], t[q_out:q_out + kv_out], t[q_out + kv_out:])
        elif key.endswith("mlp.gate_up_proj.weight"):
            base = key[: -len("gate_up_proj.weight")]
            t = out.pop(key)
            half = t.shape[0] // 2
            out[f"{base}gate_proj.weight"], out[f"{base}up_proj.weight"] = t[:half], t[half:]
        elif key.endswith("mlp.experts.gate_up_proj") and weights[key].dim() == 3:
            # stacked experts of newer checkpoints: [E, 2F, H] and [E, H, F] -> per-expert projections
            base = key[: -len("gate_up_proj")]
            t = out.pop(key)
            half = t.shape[1] // 2
            for e in range(t.shape[0]):
                out[f"{base}{e}.gate_proj.weight"], out[f"{base}{e}.up_proj.weight"] = t[e, :half], t[e, half:]
        elif key.endswith("mlp.experts.down_proj") and weights[key].dim() == 3:
            base = key[: -len("down_proj")]
            t = out.pop(key)
            for e in range(t.shape[0]):
                out[f"{base}{e}.down_proj.weight"] = t[e]
    return out


def canonical_weights(weights: dict[str, torch.Tensor], cfg: ModelConfig) -> dict[str, torch.Tensor]:
    """Strip VLM nesting prefixes and split packed projections so keys follow `model.layers.N.*`."""
    w = {}
    for k, t in weights.items():
        if k.startswith("model.language_model."):
            k = "model." + k[len("model.language_model."):]
        elif k.startswith("language_model.model."):
            k = "model." + k[len("language_model.model."):]
        elif k.startswith("language_model.lm_head."):
            k = "lm_head." + k[len("language_model.lm_head."):]
        w[k] = t
    return _split_packed(w, cfg)


class OracleLlama:
    """Generic Llama-family decoder in plain PyTorch (dense + Qwen2-MoE FFN)."""

    def __init__(self, cfg: ModelConfig, weights: dict[str, torch.Tensor], dtype: torch.dtype = torch.float32,
                 device: str | torch.device = "cpu"):
        if cfg.architecture in (Architecture.QWEN35,):
            raise LoadError(f"{cfg.architecture.value} is served by its own model class")
        self.cfg = cfg
        self.dtype = dtype
        self.device = torch.device(device)
        w = canonical_weights(weights, cfg)
        self.w = {k: v.to(device=self.device, dtype=dtype) for k, v in w.items()
                  if k.startswith(("model.embed_tokens", "model.layers.", "model.norm", "lm_head"))}
        if "model.embed_tokens.weight" not in self.w:
            raise LoadError("missing model.embed_tokens.weight")
        if "lm_head.weight" not in self.w:
            self.w["lm_head.weight"] = self.w["model.embed_tokens.weight"]  # tied
        rope = build_rope(cfg)
        self.inv_freq = torch.tensor(rope.inv_freq, dtype=torch.float32, device=self.device)
        self.rot_dim = rope.dim
        self.rope_interleaved = rope.interleaved

    # ---- cache ------------------------------------------------------------------------------
    def make_cache(self) -> ContiguousKvCache:
        return ContiguousKvCache(self.cfg.num_layers)

    # ---- building blocks ----------------------------------------------------------------------
    def _lin(self, x: torch.Tensor, base: str) -> torch.Tensor:
        y = x @ self.w[base + ".weight"].t()
        b = self.w.get(base + ".bias")
        return y + b if b is not None else y

    def _norm(self, x: torch.Tensor, key: str) -> torch.Tensor:
        return rms_norm(x, self.w[key], self.cfg.rms_norm_eps, self.cfg.norm_weight_offset)

    def _mlp(self, x: torch.Tensor, p: str) -> torch.Tensor:
        g = self._lin(x, p + ".gate_proj")
        a = torch.nn.functional.gelu(g, approximate="tanh") if self.cfg.mlp_activation == "gelu_tanh" else \
            torch.nn.functional.silu(g)
        return self._lin(a * self._lin(x, p + ".up_proj"), p + ".down_proj")

    def _moe(self, x: torch.Tensor, p: str) -> torch.Tensor:
        moe = self.cfg.moe
        shape = x.shape
        xf = x.reshape(-1, shape[-1])
        logits = xf @ self.w[p + ".gate.weight"].t()
        probs = torch.softmax(logits.float(), dim=-1)
        raw = self.cfg.raw
        if raw.get("topk_method") == "group_limited_greedy" and raw.get("n_group", 1) > 1:
            g, tg = int(raw["n_group"]), int(raw.get("topk_group", 1))      # keep only the best `topk_group` groups
            gs = probs.view(probs.shape[0], g, -1).amax(-1)
            keep = torch.zeros_like(gs).scatter_(1, gs.topk(tg, dim=-1).indices, 1.0)
            probs_sel = probs.masked_fill(keep.repeat_interleave(probs.shape[1] // g, 1) == 0, 0.0)
            topv, topi = probs_sel.topk(moe.num_experts_per_tok, dim=-1)
        else:
            topv, topi = probs.topk(moe.num_experts_per_tok, dim=-1)
        if moe.norm_topk_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        topv = topv * moe.routed_scaling_factor
        out = torch.zeros_like(xf)
        for e in range(moe.num_experts):
            sel = (topi == e)
            rows = sel.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            wgt = (topv * sel).sum(-1)[rows].to(x.dtype)
            out[rows] += self._mlp(xf[rows], f"{p}.experts.{e}") * wgt[:, None]
        if (p + ".shared_experts.gate_proj.weight") in self.w:      # DeepSeek: ungated shared experts
            out = out + self._mlp(xf, p + ".shared_experts")
        if (p + ".shared_expert.gate_proj.weight") in self.w:
            sh = self._mlp(xf, p + ".shared_expert")
            gate_key = p + ".shared_expert_gate.weight"
            if gate_key in self.w:
                sh = sh * torch.sigmoid(xf @ self.w[gate_key].t())
            out = out + sh
        return out.reshape(shape)

    def _ffn(self, x: torch.Tensor, layer: int) -> torch.Tensor:
        p = f"model.layers.{layer}.mlp"
        if (p + ".gate.weight") in self.w:
            return self._moe(x, p)
        return self._mlp(x, p)

    def _attention_mla(self, x, layer, cos, sin, cache, causal, additive_mask) -> torch.Tensor:
        """Multi-head latent attention (DeepSeek-V2; candle-llm models/llama.rs MLA path): queries optionally through
        a low-rank bottleneck, keys / values expanded from a shared compressed latent plus one rotary key head."""
        cfg, m = self.cfg, self.cfg.mla
        p = f"model.layers.{layer}.self_attn"
        B, S, _ = x.shape
        H = cfg.num_heads
        if (p + ".q_a_proj.weight") in self.w:
            q = self._lin(rms_norm(self._lin(x, p + ".q_a_proj"), self.w[p + ".q_a_layernorm.weight"], cfg.rms_norm_eps),
                          p + ".q_b_proj")
        else:
            q = self._lin(x, p + ".q_proj")
        q = q.view(B, S, H, m.q_head_dim)
        q_nope, q_pe = q[..., : m.qk_nope_head_dim], q[..., m.qk_nope_head_dim:]
        ckv = self._lin(x, p + ".kv_a_proj_with_mqa")
        c, k_pe = ckv[..., : m.kv_lora_rank], ckv[..., m.kv_lora_rank:].view(B, S, 1, m.qk_rope_head_dim)
        kv = self._lin(rms_norm(c, self.w[p + ".kv_a_layernorm.weight"], cfg.rms_norm_eps), p + ".kv_b_proj")
        kv = kv.view(B, S, H, m.qk_nope_head_dim + m.v_head_dim)
        k_nope, v = kv[..., : m.qk_nope_head_dim], kv[..., m.qk_nope_head_dim:]
        q_pe = apply_rope(q_pe, cos, sin, m.qk_rope_head_dim, True)
        k_pe = apply_rope(k_pe, cos, sin, m.qk_rope_head_dim, True)
        q = torch.cat((q_nope, q_pe), -1).transpose(1, 2)
        k = torch.cat((k_nope, k_pe.expand(B, S, H, m.qk_rope_head_dim)), -1).transpose(1, 2)
        v = v.transpose(1, 2)
        if cache is not None:
            k, v = cache.update(layer, k, v)
        o = sdpa(q, k, v, cfg.attn_scale, causal, additive_mask, None)
        return self._lin(o.transpose(1, 2).reshape(B, S, H * m.v_head_dim), p + ".o_proj")

    def _attention(self, x: torch.Tensor, layer: int, cos, sin, cache: ContiguousKvCache | None, causal: bool,
                   additive_mask) -> torch.Tensor:
        cfg = self.cfg
        if cfg.mla is not None:
            return self._attention_mla(x, layer, cos, sin, cache, causal, additive_mask)
        p = f"model.layers.{layer}.self_attn"
        B, S, _ = x.shape
        q = self._lin(x, p + ".q_proj").view(B, S, cfg.num_heads, cfg.head_dim)
        k = self._lin(x, p + ".k_proj").view(B, S, cfg.num_kv_heads, cfg.head_dim)
        v = self._lin(x, p + ".v_proj").view(B, S, cfg.num_kv_heads, cfg.head_dim)
        if (p + ".q_norm.weight") in self.w:
            q = rms_norm(q, self.w[p + ".q_norm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
            k = rms_norm(k, self.w[p + ".k_norm.weight"], cfg.rms_norm_eps, cfg.norm_weight_offset)
        q = apply_rope(q, cos, sin, self.rot_dim, self.rope_interleaved)
        k = apply_rope(k, cos, sin, self.rot_dim, self.rope_interleaved)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if cache is not None:
            k, v = cache.update(layer, k, v)
        o = sdpa(q, k, v, cfg.attn_scale, causal, additive_mask, cfg.attn_logit_softcap)
        return self._lin(o.transpose(1, 2).reshape(B, S, cfg.num_heads * cfg.head_dim), p + ".o_proj")

    def _layer(self, x, layer, cos, sin, cache, causal, additive_mask):
        p = f"model.layers.{layer}"
        attn = self._attention(self._norm(x, p + ".input_layernorm.weight"), layer, cos, sin, cache, causal,
                               additive_mask)
        if self.cfg.architecture is Architecture.GEMMA2:
            h = x + self._norm(attn, p + ".post_attention_layernorm.weight")
            f = self._ffn(self._norm(h, p + ".pre_feedforward_layernorm.weight"), layer)
            return h + self._norm(f, p + ".post_feedforward_layernorm.weight")
        if self.cfg.architecture is Architecture.GLM4:
            h = x + self._norm(attn, p + ".post_self_attn_layernorm.weight")
            f = self._ffn(self._norm(h, p + ".post_attention_layernorm.weight"), layer)
            return h + self._norm(f, p + ".post_mlp_layernorm.weight")
        h = x + attn
        return h + self._ffn(self._norm(h, p + ".post_attention_layernorm.weight"), layer)

    # ---- forwards -----------------------------------------------------------------------------
    def embed(self, ids: torch.Tensor) -> torch.Tensor:
        x = self.w["model.embed_tokens.weight"][ids]
        return x * self.cfg.embed_scale if self.cfg.embed_scale != 1.0 else x

    def hidden_states(self, ids: torch.Tensor | None, cache: ContiguousKvCache | None, offset: int = 0, *,
                      embeds: torch.Tensor | None = None, positions: torch.Tensor | None = None,
                      additive_mask: torch.Tensor | None = None, num_layers: int | None = None,
                      mrope_positions: torch.Tensor | None = None,
                      deepstack: tuple[torch.Tensor, list[torch.Tensor]] | None = None) -> torch.Tensor:
        """The residual stream after `num_layers` decoder layers (all of them by default), before the final norm.
        mrope_positions [3, S] (batch 1) replaces `positions` with the three-axis interleaved rotary table of
        Qwen3-VL; deepstack = (rows, taps) adds taps[i] to those rows of the stream after decoder layer i."""
        x = self.embed(ids.to(self.device)) if embeds is None else embeds.to(self.device, self.dtype)
        B, S, _ = x.shape
        if positions is None:
            positions = torch.arange(offset, offset + S, device=self.device)[None, :].expand(B, S)
        cos, sin = rope_cos_sin(self.inv_freq, positions.to(self.device))
        if mrope_positions is not None:
            from .qwen3_vl import interleaved_mrope_table

            cos, sin = (t[None] for t in interleaved_mrope_table(mrope_positions, self.inv_freq,
                                                                 self.cfg.mrope_section_resolved()))
        causal = additive_mask is None
        for layer in range(self.cfg.num_layers if num_layers is None else num_layers):
            x = self._layer(x, layer, cos, sin, cache, causal, additive_mask)
            if deepstack is not None and layer < len(deepstack[1]):
                x = x.clone()
                x[0, deepstack[0].to(self.device)] += deepstack[1][layer].to(self.device, x.dtype)
        return x

    def project_logits(self, h: torch.Tensor) -> torch.Tensor:
        logits = self._norm(h, "model.norm.weight") @ self.w["lm_head.weight"].t()
        c = self.cfg.final_logit_softcap
        return torch.tanh(logits / c) * c if c else logits

    @torch.no_grad()
    def decode_logits(self, ids: torch.Tensor, cache: ContiguousKvCache | None, offset: int = 0, **kw) -> torch.Tensor:
        """Logits of the last position: [B, vocab]."""
        h = self.hidden_states(ids, cache, offset, **kw)
        return self.project_logits(h[:, -1:, :])[:, 0]

    @torch.no_grad()
    def decode_logits_all(self, ids: torch.Tensor, cache: ContiguousKvCache | None, offset: int = 0, **kw
                          ) -> torch.Tensor:
        """Logits of every position: [B, S, vocab] (speculative verify)."""
        return self.project_logits(self.hidden_states(ids, cache, offset, **kw))

    @torch.no_grad()
    def generate_greedy(self, prompt: list[int], max_new_tokens: int, stop_tokens: tuple[int, ...] = ()
                        ) -> tuple[list[int], list[float]]:
        """Greedy decode (argmax, ties -> lowest index); returns tokens and the per-step top-2 logit margins."""
        cache = self.make_cache()
        ids = torch.tensor([prompt], dtype=torch.long)
        logits = self.decode_logits(ids, cache, 0)
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


def random_llama_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02, dtype: torch.dtype = torch.float32,
                         bias: bool = False) -> dict[str, torch.Tensor]:
    """N(0, std) weights (norm weights = 1) for a dense Llama-family config, HF key names."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype)

    H, D = cfg.hidden_size, cfg.head_dim
    w = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H)}
    sandwich = cfg.architecture.sandwich_norms
    one = 0.0 if cfg.architecture is Architecture.GEMMA2 else 1.0
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}"
        w[f"{p}.input_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
        w[f"{p}.post_attention_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
        if cfg.architecture is Architecture.GEMMA2:
            w[f"{p}.pre_feedforward_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
            w[f"{p}.post_feedforward_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
        elif sandwich:
            w[f"{p}.post_self_attn_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
            w[f"{p}.post_mlp_layernorm.weight"] = torch.full((H,), one, dtype=dtype)
        w[f"{p}.self_attn.q_proj.weight"] = rnd(cfg.num_heads * D, H)
        w[f"{p}.self_attn.k_proj.weight"] = rnd(cfg.num_kv_heads * D, H)
        w[f"{p}.self_attn.v_proj.weight"] = rnd(cfg.num_kv_heads * D, H)
        w[f"{p}.self_attn.o_proj.weight"] = rnd(H, cfg.num_heads * D)
        if bias:
            w[f"{p}.self_attn.q_proj.bias"] = rnd(cfg.num_heads * D)
            w[f"{p}.self_attn.k_proj.bias"] = rnd(cfg.num_kv_heads * D)
            w[f"{p}.self_attn.v_proj.bias"] = rnd(cfg.num_kv_heads * D)
        if cfg.architecture.has_qk_norm:
            w[f"{p}.self_attn.q_norm.weight"] = torch.ones(D, dtype=dtype)
            w[f"{p}.self_attn.k_norm.weight"] = torch.ones(D, dtype=dtype)
        if cfg.moe is not None and i >= cfg.moe.first_k_dense_replace:
            m = cfg.moe
            w[f"{p}.mlp.gate.weight"] = rnd(m.num_experts, H)
            for e in range(m.num_experts):
                w[f"{p}.mlp.experts.{e}.gate_proj.weight"] = rnd(m.moe_intermediate_size, H)
                w[f"{p}.mlp.experts.{e}.up_proj.weight"] = rnd(m.moe_intermediate_size, H)
                w[f"{p}.mlp.experts.{e}.down_proj.weight"] = rnd(H, m.moe_intermediate_size)
            w[f"{p}.mlp.shared_expert.gate_proj.weight"] = rnd(m.shared_expert_intermediate_size, H)
            w[f"{p}.mlp.shared_expert.up_proj.weight"] = rnd(m.shared_expert_intermediate_size, H)
            w[f"{p}.mlp.shared_expert.down_proj.weight"] = rnd(H, m.shared_expert_intermediate_size)
            w[f"{p}.mlp.shared_expert_gate.weight"] = rnd(1, H)
        else:
            w[f"{p}.mlp.gate_proj.weight"] = rnd(cfg.intermediate_size, H)
            w[f"{p}.mlp.up_proj.weight"] = rnd(cfg.intermediate_size, H)
            w[f"{p}.mlp.down_proj.weight"] = rnd(H, cfg.intermediate_size)
    w["model.norm.weight"] = torch.full((H,), one, dtype=dtype)
    if not cfg.tie_word_embeddings:
        w["lm_head.weight"] = rnd(cfg.vocab_size, H)
    return w


def tiny_llama_config() -> ModelConfig:
    """The CPU parity configuration: vocab 32000, hidden 256, 4 layers, 4/2 heads, head_dim 64, SwiGLU 688."""
    return ModelConfig(hidden_size=256, intermediate_size=688, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=64,
                       vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True)
