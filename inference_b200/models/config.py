"""Decoder configuration parsed from a Hugging Face `config.json`, with architecture dispatch.

Behavioural parity target: candle-llm/src/config.rs:16-152 (architecture dispatch), :303-533 (field
parsing and defaults), :540-596 (RoPE construction, GQA groups, attention scale).
"""
from __future__ import annotations

import enum
import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..contracts.errors import ConfigError, Unsupported


class Architecture(enum.Enum):
    LLAMA = "llama"          # Llama / Mistral / dense Qwen2 (q/k/v bias auto-detected from weights)
    QWEN3 = "qwen3"          # + per-head q/k RMSNorm
    PHI3 = "phi3"            # packed qkv_proj and gate_up_proj
    QWEN2_MOE = "qwen2_moe"  # Qwen2 attention + sparse MoE FFN with a shared expert
    GEMMA2 = "gemma2"        # (1 + w) RMSNorm, embed * sqrt(hidden), GeGLU, soft-caps, 4-norm sandwich
    GLM4 = "glm4"            # 4-norm sandwich, q/k/v bias, packed gate_up, partial interleaved RoPE
    GLM = "glm"              # GLM-4-9b (`GlmForCausalLM`): the same without the sandwich norms
    DEEPSEEK_V2 = "deepseek_v2"  # multi-head latent attention + fine-grained MoE + YaRN
    QWEN35 = "qwen3_5"       # hybrid Gated-DeltaNet / gated full attention
    QWEN3_VL = "qwen3_vl"    # VLM-wrapped Qwen3 decoder with interleaved M-RoPE

    @staticmethod
    def from_config(cfg: dict[str, Any]) -> "Architecture":
        archs = cfg.get("architectures")
        arch = archs[0] if isinstance(archs, list) and archs and isinstance(archs[0], str) else None
        model_type = cfg.get("model_type") if isinstance(cfg.get("model_type"), str) else None
        hay = f"{(arch or '').lower()} {(model_type or '').lower()}"
        if "qwen3_vl" in hay or "qwen3vl" in hay:
            return Architecture.QWEN3_VL
        if "qwen3_5" in hay or "qwen3_next" in hay:
            return Architecture.QWEN35
        if "qwen3" in hay:
            return Architecture.QWEN3
        if "qwen2_moe" in hay or "qwen2moe" in hay:
            return Architecture.QWEN2_MOE
        if "gemma2" in hay:
            return Architecture.GEMMA2
        if "glm4" in hay:
            return Architecture.GLM4
        if "glmforcausallm" in hay or model_type == "glm":
            return Architecture.GLM
        if "deepseek" in hay:
            return Architecture.DEEPSEEK_V2
        if "phi3" in hay:
            return Architecture.PHI3
        if "llama" in hay or "mistral" in hay or "qwen2" in hay or (arch is None and model_type is None):
            return Architecture.LLAMA
        raise Unsupported(f"unsupported architecture (architectures={arch!r}, model_type={model_type!r})")

    @property
    def family(self) -> str:
        return self.value

    @property
    def has_qk_norm(self) -> bool:
        return self in (Architecture.QWEN3, Architecture.QWEN3_VL)

    @property
    def rope_interleaved(self) -> bool:
        return self in (Architecture.GLM4, Architecture.GLM)

    @property
    def sandwich_norms(self) -> bool:
        return self in (Architecture.GEMMA2, Architecture.GLM4)


@dataclass(frozen=True)
class RopeScaling:
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_context: float = 8192.0


@dataclass(frozen=True)
class YarnConfig:
    factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_context: float = 4096.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0

    def softmax_mscale(self) -> float:
        return 0.1 * self.mscale_all_dim * math.log(self.factor) + 1.0 if self.factor > 1.0 else 1.0


@dataclass(frozen=True)
class MoeConfig:
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    norm_topk_prob: bool = False
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0


@dataclass(frozen=True)
class MlaConfig:
    q_lora_rank: int | None
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int

    @property
    def q_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim


@dataclass(frozen=True)
class RopeSpec:
    """Per-pair inverse frequencies plus the rotation convention."""
    inv_freq: tuple[float, ...]
    dim: int
    interleaved: bool


@dataclass
class ModelConfig:
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    architecture: Architecture = Architecture.LLAMA
    max_position_embeddings: int = 0
    quantization_bits: int | None = None
    quantization_group_size: int | None = None
    moe: MoeConfig | None = None
    attn_logit_softcap: float | None = None
    final_logit_softcap: float | None = None
    query_pre_attn_scalar: int | None = None
    partial_rotary_factor: float = 1.0
    mla: MlaConfig | None = None
    yarn: YarnConfig | None = None
    mrope_section: tuple[int, int, int] | None = None
    raw: dict[str, Any] = field(default_factory=dict, repr=False)

    # ---- parsing ---------------------------------------------------------------------------
    @staticmethod
    def from_json(top: dict[str, Any]) -> "ModelConfig":
        arch = Architecture.from_config(top)
        v = top.get("text_config", top) if arch is Architecture.QWEN3_VL else top

        def integer(key: str) -> int | None:
            x = v.get(key)
            return int(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else None

        def req(key: str) -> int:
            x = integer(key)
            if x is None:
                raise ConfigError(f"config.json missing integer `{key}`")
            return x

        def real(key: str) -> float | None:
            x = v.get(key)
            return float(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else None

        hidden = req("hidden_size")
        heads = req("num_attention_heads")
        mla = None
        if integer("kv_lora_rank") is not None:
            mla = MlaConfig(integer("q_lora_rank"), integer("kv_lora_rank"), integer("qk_nope_head_dim") or 0,
                            integer("qk_rope_head_dim") or 0, integer("v_head_dim") or hidden // heads)
        head_dim = mla.q_head_dim if mla else (integer("head_dim") or hidden // heads)
        inter = req("intermediate_size")
        tie = top.get("tie_word_embeddings")
        if not isinstance(tie, bool):
            tie = arch is Architecture.GEMMA2
        q = top.get("quantization") if isinstance(top.get("quantization"), dict) else None
        qbits = int(q["bits"]) if q and isinstance(q.get("bits"), int) and q["bits"] in (4, 8) else None
        qgroup = int(q["group_size"]) if q and isinstance(q.get("group_size"), int) else None

        moe = None
        n_exp = integer("num_experts") or integer("n_routed_experts")
        if n_exp is not None:
            moe_inter = integer("moe_intermediate_size") or inter
            shared = integer("shared_expert_intermediate_size")
            if shared is None:
                ns = integer("n_shared_experts")
                shared = ns * moe_inter if ns is not None else inter
            moe = MoeConfig(n_exp, max(1, integer("num_experts_per_tok") or n_exp), moe_inter, shared,
                            bool(v.get("norm_topk_prob", False)), real("routed_scaling_factor") or 1.0,
                            max(0, integer("first_k_dense_replace") or 0))

        # newer Hugging Face configs nest theta and the scaling block in `rope_parameters`
        rp = v.get("rope_parameters") if isinstance(v.get("rope_parameters"), dict) else None
        rs = v.get("rope_scaling") if isinstance(v.get("rope_scaling"), dict) else None
        theta = real("rope_theta")
        prf = real("partial_rotary_factor")
        if rp is not None:
            if theta is None and isinstance(rp.get("rope_theta"), (int, float)):
                theta = float(rp["rope_theta"])
            if prf is None and isinstance(rp.get("partial_rotary_factor"), (int, float)):
                prf = float(rp["partial_rotary_factor"])
            if rs is None and rp.get("rope_type", rp.get("type", "default")) not in (None, "default"):
                rs = rp
            elif rs is None and isinstance(rp.get("mrope_section"), list):
                rs = rp
        yarn, scaling, mrope = None, None, None
        if rs is not None:
            ty = rs.get("type", rs.get("rope_type"))

            def rf(key: str, default: float) -> float:
                x = rs.get(key)
                return float(x) if isinstance(x, (int, float)) and not isinstance(x, bool) else default

            if ty == "yarn":
                yarn = YarnConfig(rf("factor", 1.0), rf("beta_fast", 32.0), rf("beta_slow", 1.0),
                                  rf("original_max_position_embeddings", 4096.0), rf("mscale", 1.0),
                                  rf("mscale_all_dim", 0.0))
            ty2 = rs.get("rope_type", rs.get("type"))
            if (ty2 is None and "factor" in rs) or ty2 == "llama3":  # a bare factor block is treated as llama3
                scaling = RopeScaling(rf("factor", 1.0), rf("low_freq_factor", 1.0), rf("high_freq_factor", 4.0),
                                      rf("original_max_position_embeddings", 8192.0))
            ms = rs.get("mrope_section")
            if isinstance(ms, list) and len(ms) == 3:
                mrope = (int(ms[0]), int(ms[1]), int(ms[2]))

        return ModelConfig(
            hidden_size=hidden, intermediate_size=inter, num_layers=req("num_hidden_layers"), num_heads=heads,
            num_kv_heads=integer("num_key_value_heads") or heads, head_dim=head_dim, vocab_size=req("vocab_size"),
            rms_norm_eps=real("rms_norm_eps") or 1e-5, rope_theta=theta or 500000.0,
            rope_scaling=scaling, tie_word_embeddings=tie, architecture=arch,
            max_position_embeddings=integer("max_position_embeddings") or 0, quantization_bits=qbits,
            quantization_group_size=qgroup, moe=moe, attn_logit_softcap=real("attn_logit_softcapping"),
            final_logit_softcap=real("final_logit_softcapping"), query_pre_attn_scalar=integer("query_pre_attn_scalar"),
            partial_rotary_factor=prf or 1.0, mla=mla, yarn=yarn, mrope_section=mrope,
            raw=dict(top))

    @staticmethod
    def from_dir(path: str | Path) -> "ModelConfig":
        p = Path(path)
        p = p / "config.json" if p.is_dir() else p
        try:
            return ModelConfig.from_json(json.loads(p.read_text()))
        except json.JSONDecodeError as e:
            raise ConfigError(f"parse {p}: {e}") from e

    def to_json(self) -> dict[str, Any]:
        """A minimal HF-style config.json that round-trips through from_json."""
        d: dict[str, Any] = dict(self.raw) if self.raw else {}
        d.update({
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_layers, "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads, "head_dim": self.head_dim, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
        })
        if "model_type" not in d and "architectures" not in d:
            d["model_type"] = self.architecture.value
        if self.max_position_embeddings:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.quantization_bits:
            d["quantization"] = {"bits": self.quantization_bits}
            if self.quantization_group_size:
                d["quantization"]["group_size"] = self.quantization_group_size
        return d

    # ---- derived quantities ----------------------------------------------------------------
    @property
    def groups(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def rotary_dim(self) -> int:
        return int(round(self.head_dim * self.partial_rotary_factor)) & ~1

    @property
    def attn_scale(self) -> float:
        if self.mla is not None:
            m = self.yarn.softmax_mscale() if self.yarn else 1.0
            return self.mla.q_head_dim ** -0.5 * m * m
        return float(self.query_pre_attn_scalar or self.head_dim) ** -0.5

    @property
    def is_moe(self) -> bool:
        return self.moe is not None

    @property
    def norm_weight_offset(self) -> float:
        return 1.0 if self.architecture is Architecture.GEMMA2 else 0.0

    @property
    def embed_scale(self) -> float:
        return math.sqrt(self.hidden_size) if self.architecture is Architecture.GEMMA2 else 1.0

    @property
    def mlp_activation(self) -> str:
        return "gelu_tanh" if self.architecture is Architecture.GEMMA2 else "silu"

    def mrope_section_resolved(self) -> tuple[int, int, int]:
        if self.mrope_section:
            return tuple(max(0, s) for s in self.mrope_section)  # type: ignore[return-value]
        half = self.rotary_dim // 2
        base, rem = divmod(half, 3)
        return (base + (rem > 0), base + (rem > 1), base)


def _plain_inv_freq(dim: int, theta: float) -> list[float]:
    return [1.0 / theta ** ((2 * i) / dim) for i in range(dim // 2)]


def build_rope(cfg: ModelConfig) -> RopeSpec:
    """Inverse-frequency table for the configured RoPE variant (standard, partial / interleaved, Llama-3
    frequency-band scaling, YaRN). Parity: candle-llm/src/primitives/rope.rs:35-170, config.rs:540-575."""
    if cfg.mla is not None:
        dim = cfg.mla.qk_rope_head_dim
        if cfg.yarn is None:
            return RopeSpec(tuple(_plain_inv_freq(dim, cfg.rope_theta)), dim, True)
        y = cfg.yarn

        def correction_dim(rot: float) -> float:
            return dim * math.log(y.original_context / (rot * 2.0 * math.pi)) / (2.0 * math.log(cfg.rope_theta))

        low = max(0.0, math.floor(correction_dim(y.beta_fast)))
        high = min(float(dim - 1), math.ceil(correction_dim(y.beta_slow)))
        span = 1e-3 if abs(high - low) < 1e-3 else high - low
        out = []
        for i, extra in enumerate(_plain_inv_freq(dim, cfg.rope_theta)):
            ramp = min(1.0, max(0.0, (i - low) / span))
            out.append(extra / y.factor * ramp + extra * (1.0 - ramp))
        return RopeSpec(tuple(out), dim, True)
    rd = cfg.rotary_dim
    if rd < cfg.head_dim or cfg.architecture.rope_interleaved:
        return RopeSpec(tuple(_plain_inv_freq(rd, cfg.rope_theta)), rd, cfg.architecture.rope_interleaved)
    base = _plain_inv_freq(cfg.head_dim, cfg.rope_theta)
    rs = cfg.rope_scaling
    if rs is None:
        return RopeSpec(tuple(base), cfg.head_dim, False)
    low_wl = rs.original_context / rs.low_freq_factor
    high_wl = rs.original_context / rs.high_freq_factor
    out = []
    for inv in base:
        wl = 2.0 * math.pi / inv
        if wl > low_wl:
            out.append(inv / rs.factor)
        elif wl < high_wl:
            out.append(inv)
        else:
            smooth = (rs.original_context / wl - rs.low_freq_factor) / (rs.high_freq_factor - rs.low_freq_factor)
            out.append((1.0 - smooth) * inv / rs.factor + smooth * inv)
    return RopeSpec(tuple(out), cfg.head_dim, False)
