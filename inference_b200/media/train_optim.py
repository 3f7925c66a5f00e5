"""Optimisers and gradient utilities of the adapter trainers (candle-gen/src/train/optim.rs:20-460,
train/checkpoint.rs:7-14, train/dataset.rs:20-29).

`normalize` maps the aliases users type to the four supported optimisers by exact match (a near miss such as
"adamax" is rejected instead of silently training as Adam). Rose is a stateless range-normalised update; Prodigy
estimates its own step size `d` from the correlation between gradients and the distance travelled."""
from __future__ import annotations

import math

import torch

SUPPORTED_OPTIMIZERS = ("adamw", "adam", "rose", "prodigy")
_ALIASES = {"adamw": "adamw", "adamw8bit": "adamw", "adam8bit": "adamw", "adam": "adam", "rose": "rose",
            "roseopt": "rose", "prodigy": "prodigy", "prodigyopt": "prodigy"}


def normalize(name: str) -> str:
    s = "".join(ch for ch in name.lower() if ch.isascii() and ch.isalnum())
    return _ALIASES.get(s, s)


def is_supported(name: str) -> bool:
    return normalize(name) in SUPPORTED_OPTIMIZERS


def clip_grad_norm(grads: dict[int, torch.Tensor], params: list[torch.Tensor], max_norm: float) -> float:
    """Global L2 clipping over the gradients of `params` held in `grads` (keyed by id(param)); returns the norm
    before clipping."""
    total = 0.0
    for p in params:
        g = grads.get(id(p))
        if g is not None:
            total += float(g.double().pow(2).sum())
    norm = math.sqrt(total)
    if norm > max_norm and norm > 0:
        for p in params:
            if id(p) in grads:
                grads[id(p)] = grads[id(p)] * (max_norm / norm)
    return norm


def accumulate_grads(acc: dict[int, torch.Tensor] | None, grads: dict[int, torch.Tensor], params) -> dict:
    if acc is None:
        return dict(grads)
    for p in params:
        g = grads.get(id(p))
        if g is not None:
            acc[id(p)] = acc[id(p)] + g if id(p) in acc else g.clone()
    return acc


def scale_grads(grads: dict[int, torch.Tensor], params, factor: float) -> None:
    for p in params:
        if id(p) in grads:
            grads[id(p)] = grads[id(p)] * factor


def _zeros_to_one(t: torch.Tensor) -> torch.Tensor:
    return t + (t == 0).to(t.dtype)


class _AdamW:
    def __init__(self, params, lr, weight_decay, beta1=0.9, beta2=0.999, eps=1e-8):
        self.params, self.lr, self.wd, self.b1, self.b2, self.eps = params, lr, weight_decay, beta1, beta2, eps
        self.m = [torch.zeros_like(p) for p in params]
        self.v = [torch.zeros_like(p) for p in params]
        self.t = 0

    def step(self, grads):
        self.t += 1
        c1, c2 = 1 - self.b1 ** self.t, 1 - self.b2 ** self.t
        with torch.no_grad():
            for i, p in enumerate(self.params):
                g = grads.get(id(p))
                if g is None:
                    continue
                self.m[i].mul_(self.b1).add_(g, alpha=1 - self.b1)
                self.v[i].mul_(self.b2).addcmul_(g, g, value=1 - self.b2)
                p.mul_(1 - self.lr * self.wd)
                p.addcdiv_(self.m[i] / c1, (self.v[i] / c2).sqrt() + self.eps, value=-self.lr)


class Rose:
    """Stateless: each row's gradient is centred and divided by its range (max - min), with the ranges pulled
    toward their mean by a trust factor mean / (std + mean)."""

    def __init__(self, params, lr: float, weight_decay: float, centralize: bool = True, stabilize: bool = True):
        self.params, self.base_lr, self.lr, self.wd = params, lr, lr, weight_decay
        self.centralize, self.stabilize = centralize, stabilize

    def set_lr_scaled(self, mult: float) -> None:
        self.lr = self.base_lr * mult

    def update_one(self, param: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
        lr = self.lr
        p = param * max(0.0, 1.0 - lr * self.wd) if self.wd != 0 else param.clone()
        if grad.dim() == 0:
            raise ValueError("Rose: 0-D parameters are unsupported (adapter factors are matrices)")
        if grad.dim() == 1:
            denom = _zeros_to_one(grad.max().abs() - grad.min())
            return p + grad / denom * (-lr)
        g2 = grad.reshape(grad.shape[0], -1)
        if self.centralize:
            g2 = g2 - g2.mean(-1, keepdim=True)
        raw = g2.max(-1, keepdim=True).values.abs() - g2.min(-1, keepdim=True).values
        if self.stabilize:
            mean = raw.mean()
            std = (raw - mean).pow(2).mean().sqrt()
            trust = mean / _zeros_to_one(std + mean)
            denom = (raw - mean) * trust + mean
        else:
            denom = raw
        return p + (g2 / _zeros_to_one(denom) * (-lr)).reshape(grad.shape)

    def step(self, grads) -> None:
        with torch.no_grad():
            for p in self.params:
                g = grads.get(id(p))
                if g is not None:
                    p.copy_(self.update_one(p, g))


class Prodigy:
    def __init__(self, params, lr: float, weight_decay: float):
        use_lr = lr if lr >= 0.1 else 1.0          # Prodigy's lr is a multiplier on its own estimate; tiny values mean "default"
        self.params, self.base_lr, self.lr, self.wd = params, use_lr, use_lr, weight_decay
        self.beta1, self.beta2 = 0.9, 0.999
        self.beta3 = math.sqrt(self.beta2)
        self.eps, self.d, self.d0, self.d_max = 1e-6, 1e-6, 1e-6, 1e-6
        self.d_numerator, self.d_coef, self.growth_rate = 0.0, 1.0, math.inf
        self.state: dict[int, dict[str, torch.Tensor]] = {}

    def set_lr_scaled(self, mult: float) -> None:
        self.lr = self.base_lr * mult

    def step(self, grads) -> None:
        b1, b2, b3 = self.beta1, self.beta2, self.beta3
        d, d0, lr, eps = self.d, self.d0, self.lr, self.eps
        dlr = d * lr
        d_num = self.d_numerator * b3
        dn_scale = (d / d0) * dlr
        delta_num, d_denom, seen = 0.0, 0.0, False
        with torch.no_grad():
            for i, p in enumerate(self.params):
                g = grads.get(id(p))
                if g is None:
                    continue
                seen = True
                st = self.state.setdefault(i, {"exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p),
                                               "s": torch.zeros_like(p), "p0": p.detach().clone()})
                delta_num += float((g * (st["p0"] - p)).sum().double()) * dn_scale
                st["exp_avg"] = st["exp_avg"] * b1 + g * (d * (1 - b1))
                st["exp_avg_sq"] = st["exp_avg_sq"] * b2 + g * g * (d * d * (1 - b2))
                st["s"] = st["s"] * b3 + g * dn_scale
                d_denom += float(st["s"].abs().sum().double())
            if not seen or d_denom == 0.0:
                return
            g_num = d_num + delta_num
            d_hat = self.d_coef * g_num / d_denom
            d_new = max(d, d_hat) if d == d0 else d
            d_max = max(self.d_max, d_hat)
            d_new = min(d_max, d_new * self.growth_rate)
            self.d_numerator, self.d, self.d_max = g_num, d_new, d_max
            for i, p in enumerate(self.params):
                if grads.get(id(p)) is None:
                    continue
                st = self.state[i]
                denom = st["exp_avg_sq"].sqrt() + d_new * eps
                if self.wd != 0:
                    p.mul_(1 - self.wd * dlr)
                p.sub_(st["exp_avg"] / denom * dlr)


class TrainOptimizer:
    """AdamW / Adam / Rose / Prodigy behind one `step(grads)` + `set_lr_scaled(mult)` surface."""

    def __init__(self, name: str, params: list[torch.Tensor], lr: float, weight_decay: float):
        kind = normalize(name)
        if kind == "adamw":
            self.inner = _AdamW(params, lr, weight_decay)
        elif kind == "adam":
            self.inner = _AdamW(params, lr, 0.0)
        elif kind == "rose":
            self.inner = Rose(params, lr, weight_decay)
        elif kind == "prodigy":
            self.inner = Prodigy(params, lr, weight_decay)
        else:
            raise ValueError(f"unsupported optimizer {kind!r}; supported: {', '.join(SUPPORTED_OPTIMIZERS)}")
        self.kind, self.base_lr = kind, lr

    def set_lr_scaled(self, mult: float) -> None:
        if isinstance(self.inner, _AdamW):
            self.inner.lr = self.base_lr * mult
        else:
            self.inner.set_lr_scaled(mult)

    def step(self, grads: dict[int, torch.Tensor]) -> None:
        self.inner.step(grads)


def grads_of(loss: torch.Tensor, params: list[torch.Tensor]) -> dict[int, torch.Tensor]:
    gs = torch.autograd.grad(loss, params, allow_unused=True)
    return {id(p): g for p, g in zip(params, gs) if g is not None}


def file_stem(file_name: str) -> str:
    return file_name[: -len(".safetensors")] if file_name.endswith(".safetensors") else file_name


def checkpoint_filename(stem: str, step: int) -> str:
    """Zero-padded so intermediate checkpoints sort by step."""
    return f"{stem}-step{step:06d}.safetensors"


def bucket_resolution(resolution: int) -> int:
    """Training edge snapped down to a multiple of 32 (0 means the 512 default)."""
    return 512 if resolution == 0 else max(32, resolution // 32 * 32)


def checkpointed_backward(segments, x: torch.Tensor, loss_fn, params: list[torch.Tensor]) -> tuple[float, dict]:
    """Manual gradient checkpointing (candle-gen/src/train/gradient_checkpoint.rs:64-122): the forward keeps only
    each segment's input; the backward recomputes one segment at a time and chains the input gradient, so peak
    activation memory is one segment's instead of the whole stack's. Returns (loss value, grads by id(param))."""
    inputs = []
    h = x
    with torch.no_grad():
        for seg in segments:
            inputs.append(h)
            h = seg(h)
    out = h.detach().requires_grad_(True)
    loss = loss_fn(out)
    (g_out,) = torch.autograd.grad(loss, out)
    grads: dict[int, torch.Tensor] = {}
    for seg, inp in zip(reversed(segments), reversed(inputs)):
        xin = inp.detach().requires_grad_(True)
        y = seg(xin)
        live = [p for p in params if p.requires_grad]
        gs = torch.autograd.grad(y, [xin] + live, grad_outputs=g_out, allow_unused=True)
        g_out = gs[0]
        for p, g in zip(live, gs[1:]):
            if g is not None:
                grads[id(p)] = grads[id(p)] + g if id(p) in grads else g
    return float(loss.detach()), grads
