"""Additive adapters on a frozen linear layer: LoRA and structured LoKr residuals, and the dense weight deltas of
LoKr / LoHa files for merging (candle-gen/src/quant/adapt.rs:136-610, train/lora.rs:809-914, train/merge.rs:401-500).

y = base(x) + sum_i scale_i * ((x A_i^T) B_i^T) + sum_j lokr_j(x). The base may be a dense bf16 weight or any
packed weight (`ops.quant.QuantWeight`, `ops.nvfp4.Nvfp4Linear`): adapters never touch the packed bytes. A LoKr
residual is evaluated without forming the Kronecker product: with W = w1 (a x c) (x) w2 (b x d),
y[n, i*b + j] = sum_p w1[i, p] * (x[n, p, :] . w2[j, :])."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


def _factor(full, a, b, name: str) -> torch.Tensor:
    if full is not None:
        return full.float()
    if a is not None and b is not None:
        return a.float() @ b.float()
    raise ValueError(f"lokr: {name} missing (need full lokr_{name} or lokr_{name}_a . lokr_{name}_b)")


def reconstruct_lokr_delta(w1=None, w1_a=None, w1_b=None, w2=None, w2_a=None, w2_b=None, *, alpha: float = 1.0,
                           rank: float = 1.0, scale: float = 1.0, base_shape: tuple[int, int]) -> torch.Tensor:
    """Dense delta kron(w1, w2) * (alpha / rank) * scale, shaped like the base weight [out, in]."""
    f1, f2 = _factor(w1, w1_a, w1_b, "w1"), _factor(w2, w2_a, w2_b, "w2")
    return torch.kron(f1, f2).reshape(base_shape) * ((alpha / rank) * scale)


def reconstruct_loha_delta(w1_a, w1_b, w2_a, w2_b, scale: float, base_shape: tuple[int, int]) -> torch.Tensor:
    """Dense delta (w1_a w1_b) * (w2_a w2_b) (Hadamard product of two low-rank matrices) * scale."""
    return ((w1_a.float() @ w1_b.float()) * (w2_a.float() @ w2_b.float())).reshape(base_shape) * scale


@dataclass
class LokrFactors:
    w1: torch.Tensor        # [a, c] fp32
    w2: torch.Tensor        # [b, d] fp32, pre-multiplied by the adapter scale
    a: int
    b: int
    c: int
    d: int

    @classmethod
    def build(cls, scale: float, base_shape: tuple[int, int], w1=None, w1_a=None, w1_b=None, w2=None, w2_t2=None,
              w2_a=None, w2_b=None) -> "LokrFactors | None":
        """None when the factors cannot be applied in structured form (Tucker core present, non-matrix factors,
        or a Kronecker shape that does not tile the base): the caller then folds a dense delta instead."""
        if w2_t2 is not None:
            return None
        f1, f2 = _factor(w1, w1_a, w1_b, "w1"), _factor(w2, w2_a, w2_b, "w2")
        if f1.dim() != 2 or f2.dim() != 2:
            return None
        (a, c), (b, d) = f1.shape, f2.shape
        if a * b != base_shape[0] or c * d != base_shape[1]:
            return None
        return cls(f1.contiguous(), (f2 * scale).contiguous(), a, b, c, d)

    def to(self, device) -> "LokrFactors":
        return LokrFactors(self.w1.to(device), self.w2.to(device), self.a, self.b, self.c, self.d)

    def residual(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        n = max(1, x.numel() // x.shape[-1])
        t = (x.reshape(n * self.c, self.d) @ self.w2.to(x.dtype).t()).reshape(n, self.c, self.b)
        y = self.w1.to(x.dtype).reshape(1, self.a, self.c) @ t                  # [n, a, b]
        return y.reshape(*lead, self.a * self.b)


@dataclass
class ThirdPartyLokr:
    """One module's tensors from a LyCORIS LoKr file."""
    w1: torch.Tensor | None = None
    w1_a: torch.Tensor | None = None
    w1_b: torch.Tensor | None = None
    w2: torch.Tensor | None = None
    w2_a: torch.Tensor | None = None
    w2_b: torch.Tensor | None = None
    alpha: float | None = None

    def rank(self) -> float | None:
        if self.w1_a is not None:
            return float(self.w1_a.shape[1])
        return float(self.w2_a.shape[1]) if self.w2_a is not None else None

    def lycoris_scale(self) -> float:
        r = self.rank()
        return 1.0 if r is None else (self.alpha if self.alpha is not None else r) / r

    def delta(self, base_shape: tuple[int, int], user_scale: float) -> torch.Tensor:
        return reconstruct_lokr_delta(self.w1, self.w1_a, self.w1_b, self.w2, self.w2_a, self.w2_b,
                                      alpha=self.lycoris_scale(), rank=1.0, scale=user_scale, base_shape=base_shape)


@dataclass
class ThirdPartyLoha:
    w1_a: torch.Tensor | None = None
    w1_b: torch.Tensor | None = None
    w2_a: torch.Tensor | None = None
    w2_b: torch.Tensor | None = None
    alpha: float | None = None

    def lycoris_scale(self) -> float:
        if self.w1_b is None:
            return 1.0
        r = float(self.w1_b.shape[0])
        return (self.alpha if self.alpha is not None else r) / r

    def delta(self, base_shape: tuple[int, int], user_scale: float) -> torch.Tensor:
        if any(t is None for t in (self.w1_a, self.w1_b, self.w2_a, self.w2_b)):
            raise ValueError("loha: a hada_w1/w2 a/b factor is missing")
        return reconstruct_loha_delta(self.w1_a, self.w1_b, self.w2_a, self.w2_b, self.lycoris_scale() * user_scale,
                                      base_shape)


def parse_thirdparty(tensors: dict[str, torch.Tensor]) -> tuple[dict[str, ThirdPartyLokr], dict[str, ThirdPartyLoha]]:
    """Groups `<module>.lokr_w1[_a|_b]`, `.lokr_w2[_a|_b]`, `.hada_w1_a` ... and `.alpha` keys by module."""
    lokr: dict[str, ThirdPartyLokr] = {}
    loha: dict[str, ThirdPartyLoha] = {}
    alphas = {k[: -len(".alpha")]: float(v.flatten()[0]) for k, v in tensors.items() if k.endswith(".alpha")}
    for k, v in tensors.items():
        mod, _, leaf = k.rpartition(".")
        if leaf.startswith("lokr_") and leaf[5:] in ("w1", "w1_a", "w1_b", "w2", "w2_a", "w2_b"):
            setattr(lokr.setdefault(mod, ThirdPartyLokr(alpha=alphas.get(mod))), leaf[5:], v)
        elif leaf.startswith("hada_") and leaf[5:] in ("w1_a", "w1_b", "w2_a", "w2_b"):
            setattr(loha.setdefault(mod, ThirdPartyLoha(alpha=alphas.get(mod))), leaf[5:], v)
    return lokr, loha


@dataclass
class AdaptLinear:
    """A base linear (dense weight [out, in] or a packed layer exposing `__call__`) plus additive adapters."""
    base: object
    in_features: int
    out_features: int
    bias: torch.Tensor | None = None
    loras: list[tuple[torch.Tensor, torch.Tensor, float]] = field(default_factory=list)   # (A [r,in], B [out,r], s)
    lokrs: list[LokrFactors] = field(default_factory=list)

    @classmethod
    def from_dense(cls, weight: torch.Tensor, bias: torch.Tensor | None = None) -> "AdaptLinear":
        return cls(weight, weight.shape[1], weight.shape[0], bias)

    @classmethod
    def from_packed(cls, layer, in_features: int, out_features: int) -> "AdaptLinear":
        return cls(layer, in_features, out_features)

    def is_packed(self) -> bool:
        return not isinstance(self.base, torch.Tensor)

    def is_adapted(self) -> bool:
        return bool(self.loras or self.lokrs)

    def push_lora(self, a: torch.Tensor, b: torch.Tensor, scale: float) -> None:
        assert a.shape[1] == self.in_features and b.shape[0] == self.out_features and a.shape[0] == b.shape[1]
        self.loras.append((a, b, float(scale)))

    def push_lokr_structured(self, factors: LokrFactors) -> None:
        assert factors.a * factors.b == self.out_features and factors.c * factors.d == self.in_features
        self.lokrs.append(factors)

    def clear_adapters(self) -> None:
        self.loras.clear()
        self.lokrs.clear()

    def _base(self, x: torch.Tensor) -> torch.Tensor:
        if self.is_packed():
            return self.base(x)
        w = self.base
        if x.is_cuda and w.dtype == torch.bfloat16 and x.dtype == torch.bfloat16:
            from ..ops import linear

            return linear(x, w, self.bias)
        y = x @ w.to(x.dtype).t()
        return y + self.bias.to(x.dtype) if self.bias is not None else y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._base(x)
        for a, b, s in self.loras:
            y = y + ((x @ a.to(x.dtype).t()) @ b.to(x.dtype).t()) * s
        for f in self.lokrs:
            y = y + f.residual(x)
        return y

    __call__ = forward

    def merged_weight(self) -> torch.Tensor:
        """Dense fp32 weight with every adapter folded in (dense bases only)."""
        if self.is_packed():
            raise ValueError("merged_weight needs a dense base")
        w = self.base.float().clone()
        for a, b, s in self.loras:
            w += (b.float() @ a.float()) * s
        for f in self.lokrs:
            w += torch.kron(f.w1, f.w2).reshape(w.shape)
        return w
