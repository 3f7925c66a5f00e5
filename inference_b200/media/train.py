"""LoRA adapter training for flow-matching DiTs and adapter merging at load time (the role of
candle-gen/src/train/flow_match.rs:296-680 and train/lora.rs: cached latents + text embeddings, frozen DiT with
low-rank adapters on the attention / MLP projections, logit-normal timestep sampling, x_t = (1 - t) x0 + t eps,
target velocity eps - x0, AdamW with gradient accumulation and clipping, periodic checkpoints with resume, PEFT-style
adapter files).

Training differentiates through the plain-PyTorch model (`OracleFluxDiT.forward_grad`) on whatever device its weights
live on; it is outside the serving hot path. Dataset: a directory of `*.safetensors` items with `latent`
[16, h, w] (already scaled VAE latents), `txt` [L, context_dim] and `pooled` [vec_dim]."""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.traits import SimpleDescriptor, Trainer, TrainingConfig, TrainingProgress
from ..io.safetensors_io import load_file, save_file
from ..models.dit_flux import FluxConfig, OracleFluxDiT, make_ids
from .flux import patchify

TARGET_SUFFIXES = ("img_attn.qkv", "img_attn.proj", "txt_attn.qkv", "txt_attn.proj", "linear1", "linear2")


def lr_at(schedule: str, step: int, total: int, warmup: int, base: float) -> float:
    """constant | linear | cosine, each with linear warm-up (gen-core/src/train/schedule.rs:12-59)."""
    if warmup > 0 and step < warmup:
        return base * (step + 1) / warmup
    if schedule == "constant":
        return base
    frac = (step - warmup) / max(1, total - warmup)
    if schedule == "linear":
        return base * max(0.0, 1.0 - frac)
    if schedule == "cosine":
        return base * 0.5 * (1.0 + math.cos(math.pi * min(1.0, frac)))
    raise InferenceError(f"unknown lr_schedule {schedule!r} (constant | linear | cosine)")


ADAPTER_KEYS = {2: ("lora_A.weight", "lora_B.weight"), 3: ("lokr_w1", "lokr_w2_a", "lokr_w2_b")}


def kron_split(n: int) -> tuple[int, int]:
    """(small, large) with small * large == n and small the largest divisor not above sqrt(n)."""
    m = int(math.isqrt(n))
    while n % m:
        m -= 1
    return m, n // m


def lora_targets(weights: dict[str, torch.Tensor], suffixes: tuple[str, ...] = TARGET_SUFFIXES) -> list[str]:
    names = sorted({k[: -len(".weight")] for k in weights if k.endswith(".weight") and weights[k].dim() == 2})
    return [n for n in names if n.endswith(suffixes)]


def merge_lora(weights: dict[str, torch.Tensor], adapter: dict[str, torch.Tensor], scale: float = 1.0,
               prefix: str = "transformer.") -> dict[str, torch.Tensor]:
    """W += scale * (alpha / r) * B A for every `<prefix><module>.lora_A.weight` / `.lora_B.weight` pair; a per-module
    `<module>.alpha` scalar (kohya style) overrides alpha = r."""
    out = dict(weights)
    mods = sorted({k[len(prefix): -len(".lora_A.weight")] for k in adapter if k.startswith(prefix) and
                   k.endswith(".lora_A.weight")})
    for m in mods:
        a, b = adapter[f"{prefix}{m}.lora_A.weight"].float(), adapter[f"{prefix}{m}.lora_B.weight"].float()
        key = m + ".weight"
        if key not in out:
            raise LoadError(f"adapter targets '{m}', which the model does not have")
        r = a.shape[0]
        alpha = float(adapter[f"{prefix}{m}.alpha"]) if f"{prefix}{m}.alpha" in adapter else float(r)
        w = out[key]
        out[key] = (w.float() + (b @ a) * (scale * alpha / r)).to(w.dtype)
    return out


class FluxLoraTrainer(Trainer):
    family, target_suffixes, item_keys = "flux", TARGET_SUFFIXES, ("latent", "txt", "pooled")

    def __init__(self, cfg: FluxConfig, weights: dict[str, torch.Tensor], backend: str = "cpu", device="cpu"):
        self.cfg, self.backend, self.device = cfg, backend, torch.device(device)
        self.model = OracleFluxDiT(cfg, weights, dtype=torch.float32, device=self.device)
        for t in self.model.w.values():
            t.requires_grad_(False)

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor("flux1_lora_trainer" if self.backend != "cpu" else "cpu_flux1_lora_trainer", "flux",
                                self.backend, {"adapters": ["lora", "lokr"], "targets": list(TARGET_SUFFIXES)})

    def validate(self, c: TrainingConfig) -> None:
        if c.adapter not in ("lora", "lokr"):
            raise InferenceError(f"adapter kind {c.adapter!r} is not supported (lora, lokr)")
        if c.dataset_dir is None or not Path(c.dataset_dir).is_dir():
            raise InferenceError("dataset_dir must be an existing directory of cached items")
        if c.output_dir is None:
            raise InferenceError("output_dir is required")
        if c.steps < 1 or c.rank < 1 or c.batch_size != 1 or c.grad_accum < 1 or c.learning_rate <= 0:
            raise InferenceError("steps, rank, grad_accum must be >= 1, batch_size == 1, learning_rate > 0")
        lr_at(c.lr_schedule, 0, c.steps, c.warmup_steps, c.learning_rate)

    # ---- pieces ------------------------------------------------------------------------------------------
    def _items(self, d: Path) -> list[dict[str, torch.Tensor]]:
        files = sorted(Path(d).glob("*.safetensors"))
        if not files:
            raise InferenceError(f"{d}: no dataset items (*.safetensors with latent / txt / pooled)")
        items = []
        for f in files:
            t = load_file(f)
            if not set(self.item_keys) <= set(t):
                raise InferenceError(f"{f}: needs tensors {', '.join(self.item_keys)}")
            items.append({k: v.float().to(self.device) for k, v in t.items()})
        return items

    def _init_adapters(self, rank: int, gen: torch.Generator, kind: str = "lora") -> dict[str, list[torch.Tensor]]:
        """LoRA: [A [r, in] ~ N(0, 1 / in), B [out, r] = 0]. LoKr (candle-gen/src/train/lokr.rs; LyCORIS layout): the
        delta is kron(w1 [a, c], w2_a [b, r] w2_b [r, d]) with out = a b, in = c d split at the divisor nearest the
        square root (small factor first); w1 and w2_a start random, w2_b at zero, so training starts from the base."""
        ad = {}
        for name in lora_targets(self.model.w, self.target_suffixes):
            w = self.model.w[name + ".weight"]
            if kind == "lora":
                a = (torch.randn(rank, w.shape[1], generator=gen) / math.sqrt(w.shape[1])).to(self.device).requires_grad_()
                b = torch.zeros(w.shape[0], rank, device=self.device, requires_grad=True)
                ad[name] = [a, b]
                continue
            (oa, ob), (ic, idd) = kron_split(w.shape[0]), kron_split(w.shape[1])
            r = max(1, min(rank, ob, idd))
            w1 = (torch.randn(oa, ic, generator=gen) / math.sqrt(ic)).to(self.device).requires_grad_()
            w2a = (torch.randn(ob, r, generator=gen) / math.sqrt(r)).to(self.device).requires_grad_()
            w2b = torch.zeros(r, idd, device=self.device, requires_grad=True)
            ad[name] = [w1, w2a, w2b]
        return ad

    def loss_on(self, item, t: float, noise: torch.Tensor) -> torch.Tensor:
        """Flow-matching loss of one item at time t with the given noise: || v_theta(x_t, t) - (eps - x0) ||^2."""
        x0 = patchify(item["latent"][None])
        eps = patchify(noise[None])
        xt = (1.0 - t) * x0 + t * eps
        lh, lw = item["latent"].shape[1] // 2, item["latent"].shape[2] // 2
        txt_ids, img_ids = make_ids(lh, lw, item["txt"].shape[0], self.device)
        g = torch.full((1,), 3.5, device=self.device) if self.cfg.guidance_embed else None
        v = self.model.forward_grad(xt, img_ids, item["txt"][None], txt_ids, torch.full((1,), t, device=self.device),
                                    item["pooled"][None], g)
        return torch.mean((v - (eps - x0)) ** 2)

    # ---- contract ------------------------------------------------------------------------------------------
    def train(self, c: TrainingConfig, on_progress: Callable[[TrainingProgress], None] = lambda p: None) -> Path:
        self.validate(c)
        out_dir = Path(c.output_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        items = self._items(Path(c.dataset_dir))
        gen = torch.Generator().manual_seed(c.seed)
        adapters = self._init_adapters(c.rank, gen, c.adapter)
        params = [p for ab in adapters.values() for p in ab]
        opt = torch.optim.AdamW(params, lr=c.learning_rate, weight_decay=0.0)
        start = 0
        if c.resume is not None:
            start = self._load_checkpoint(Path(c.resume), adapters, opt, gen)
        scale = c.alpha / c.rank
        self.model.lora = {n: (*ts, (c.alpha / ts[1].shape[1]) if len(ts) == 3 else scale) for n, ts in adapters.items()}
        last = None
        try:
            for step in range(start, c.steps):
                if c.cancel.is_cancelled():
                    raise Canceled(f"training cancelled at step {step}")
                lr = lr_at(c.lr_schedule, step, c.steps, c.warmup_steps, c.learning_rate)
                for gparam in opt.param_groups:
                    gparam["lr"] = lr
                opt.zero_grad(set_to_none=True)
                total = 0.0
                for micro in range(c.grad_accum):
                    item = items[(step * c.grad_accum + micro) % len(items)]
                    u = torch.randn(1, generator=gen).item()
                    t = 1.0 / (1.0 + math.exp(-u))                      # logit-normal(0, 1)
                    noise = torch.randn(item["latent"].shape, generator=gen).to(self.device)
                    loss = self.loss_on(item, t, noise) / c.grad_accum
                    loss.backward()
                    total += float(loss.detach())
                torch.nn.utils.clip_grad_norm_(params, 1.0)
                opt.step()
                ck = None
                if c.save_every and (step + 1) % c.save_every == 0 and step + 1 < c.steps:
                    ck = self._save(out_dir / f"adapter-step{step + 1:06d}.safetensors", adapters, c, step + 1, opt, gen)
                on_progress(TrainingProgress(step + 1, c.steps, total, lr, ck))
            last = self._save(out_dir / "adapter.safetensors", adapters, c, c.steps, opt, gen)
        finally:
            self.model.lora = None
        return last

    # ---- checkpoints ---------------------------------------------------------------------------------------
    def _save(self, path: Path, adapters, c: TrainingConfig, step: int, opt, gen) -> Path:
        t = {}
        for n, ts in adapters.items():
            for key, v in zip(ADAPTER_KEYS[len(ts)], ts):
                t[f"transformer.{n}.{key}"] = v.detach().cpu().contiguous()
            if len(ts) == 3:
                t[f"transformer.{n}.alpha"] = torch.tensor(float(c.alpha))
        fmt = "peft-lora" if c.adapter == "lora" else "lycoris-lokr"
        save_file(t, path, metadata={"format": fmt, "rank": str(c.rank), "alpha": str(c.alpha),
                                     "step": str(step), "base": self.family})
        state = {"rng": gen.get_state()}
        for i, p in enumerate(opt.param_groups[0]["params"]):
            st = opt.state.get(p, {})
            if st:
                state[f"exp_avg.{i}"] = st["exp_avg"].detach().cpu().contiguous()
                state[f"exp_avg_sq.{i}"] = st["exp_avg_sq"].detach().cpu().contiguous()
                state[f"step.{i}"] = st["step"].detach().cpu().reshape(1).float() if torch.is_tensor(st["step"]) \
                    else torch.tensor([float(st["step"])])
        save_file(state, path.with_suffix(".state.safetensors"), metadata={"step": str(step)})
        return path

    def _load_checkpoint(self, path: Path, adapters, opt, gen) -> int:
        from ..io.safetensors_io import SafetensorsFile

        if not path.is_file():
            raise LoadError(f"resume checkpoint {path} not found")
        t = load_file(path)
        for n, ts in adapters.items():
            for key, v in zip(ADAPTER_KEYS[len(ts)], ts):
                v.data.copy_(t[f"transformer.{n}.{key}"])
        sp = path.with_suffix(".state.safetensors")
        f = SafetensorsFile(sp)
        step = int(f.metadata.get("step", "0")) if hasattr(f, "metadata") else 0
        f.close()
        st = load_file(sp)
        gen.set_state(st["rng"].to(torch.uint8))
        for i, p in enumerate(opt.param_groups[0]["params"]):
            if f"exp_avg.{i}" in st:
                opt.state[p] = {"exp_avg": st[f"exp_avg.{i}"].to(p.device), "exp_avg_sq": st[f"exp_avg_sq.{i}"].to(p.device),
                                "step": st[f"step.{i}"].reshape(()).to(torch.float32)}
        return step


Z_IMAGE_TARGETS = ("attention.to_q", "attention.to_k", "attention.to_v", "attention.to_out.0")


class ZImageLoraTrainer(FluxLoraTrainer):
    """The same loop on the Z-Image DiT (candle-gen-z-image/src/training.rs): adapters on the four attention projections
    of every block; the model is conditioned on 1 - t and its output is negated to give the velocity. Items hold
    `latent` [16, h, w] and `txt` [L, cap_feat_dim] (the caption encoder's features)."""
    family, target_suffixes, item_keys = "z-image", Z_IMAGE_TARGETS, ("latent", "txt")

    def __init__(self, cfg, weights: dict[str, torch.Tensor], backend: str = "cpu", device="cpu"):
        from ..models.dit_zimage import OracleZImageDiT

        self.cfg, self.backend, self.device = cfg, backend, torch.device(device)
        self.model = OracleZImageDiT(cfg, weights, dtype=torch.float32, device=self.device)
        for t in self.model.w.values():
            t.requires_grad_(False)

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor("z_image_lora_trainer" if self.backend != "cpu" else "cpu_z_image_lora_trainer",
                                "z-image", self.backend, {"adapters": ["lora"], "targets": list(Z_IMAGE_TARGETS)})

    def loss_on(self, item, t: float, noise: torch.Tensor) -> torch.Tensor:
        x0, eps = item["latent"][None], noise[None]
        xt = (1.0 - t) * x0 + t * eps
        out = self.model.forward_grad(xt, torch.full((1,), 1.0 - t, device=self.device), item["txt"][None])
        return torch.mean((-out - (eps - x0)) ** 2)


def z_image_trainer_registration(backend: str):
    """`z_image_lora_trainer` (kind "trainer"): loads the DiT of a Z-Image snapshot directory."""
    from ..contracts.gen_core.registry import Registration
    from ..contracts.gen_core.runtime import LoadSpec

    tid = "z_image_lora_trainer" if backend != "cpu" else "cpu_z_image_lora_trainer"

    def load(spec: LoadSpec) -> ZImageLoraTrainer:
        from ..io.safetensors_io import load_dir
        from .z_image import ZImagePipeline, ZImageVariant

        if spec.weights is None or spec.weights.is_file:
            raise InferenceError(f"{tid}: needs a snapshot directory")
        root = Path(spec.weights.path)
        device = torch.device("cuda", torch.cuda.current_device()) if backend != "cpu" else torch.device("cpu")
        if not (root / "transformer").is_dir():
            raise LoadError(f"{tid}: missing {root / 'transformer'}")
        pipe = ZImagePipeline(ZImageVariant.BASE, root, "cpu", device)
        return ZImageLoraTrainer(pipe.dit_cfg, load_dir(root / "transformer"), backend, device)

    return Registration(descriptor=lambda: SimpleDescriptor(tid, "z-image", backend, {"adapters": ["lora"]}), load=load)


WAN_TARGETS = ("attn1.to_q", "attn1.to_k", "attn1.to_v", "attn1.to_out.0", "attn2.to_q", "attn2.to_k", "attn2.to_v",
               "attn2.to_out.0")


class WanLoraTrainer(FluxLoraTrainer):
    """The same loop on one Wan expert (candle-gen-wan/src/training.rs): adapters on the self- and cross-attention
    projections; x_t = (1 - t) x0 + t eps, the model sees the timestep 1000 t and predicts the velocity eps - x0. Items
    hold `latent` [16, T, h, w] (normalised video latents; T = 1 for stills) and `txt` [L, text_dim]."""
    family, target_suffixes, item_keys = "wan", WAN_TARGETS, ("latent", "txt")

    def __init__(self, cfg, weights: dict[str, torch.Tensor], backend: str = "cpu", device="cpu"):
        from ..models.dit_wan import WanDiT

        self.cfg, self.backend, self.device = cfg, backend, torch.device(device)
        self.model = WanDiT(cfg, weights, dtype=torch.float32, device=self.device)
        for t in self.model.w.values():
            t.requires_grad_(False)

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor("wan_lora_trainer" if self.backend != "cpu" else "cpu_wan_lora_trainer", "wan", self.backend,
                                {"adapters": ["lora"], "targets": list(WAN_TARGETS)})

    def loss_on(self, item, t: float, noise: torch.Tensor) -> torch.Tensor:
        x0, eps = item["latent"][None], noise[None]
        xt = (1.0 - t) * x0 + t * eps
        out = self.model.forward_grad(xt, torch.full((1,), 1000.0 * t, device=self.device), item["txt"][None])
        return torch.mean((out - (eps - x0)) ** 2)


def wan_trainer_registration(backend: str):
    """`wan_lora_trainer` (kind "trainer"): loads one expert of a Wan snapshot directory (`transformer/` unless the load
    spec's components name another sub-directory)."""
    from ..contracts.gen_core.registry import Registration
    from ..contracts.gen_core.runtime import LoadSpec

    tid = "wan_lora_trainer" if backend != "cpu" else "cpu_wan_lora_trainer"

    def load(spec: LoadSpec) -> WanLoraTrainer:
        from ..io.safetensors_io import load_dir
        from .wan import WanPipeline

        if spec.weights is None or spec.weights.is_file:
            raise InferenceError(f"{tid}: needs a snapshot directory")
        root = Path(spec.weights.path)
        device = torch.device("cuda", torch.cuda.current_device()) if backend != "cpu" else torch.device("cpu")
        if not (root / "transformer").is_dir():
            raise LoadError(f"{tid}: missing {root / 'transformer'}")
        pipe = WanPipeline(root, "cpu", device)
        return WanLoraTrainer(pipe.dit_cfg, load_dir(root / "transformer"), backend, device)

    return Registration(descriptor=lambda: SimpleDescriptor(tid, "wan", backend, {"adapters": ["lora"]}), load=load)


KREA_TARGETS = ("attn.to_q", "attn.to_k", "attn.to_v", "attn.to_out.0")


class KreaLoraTrainer(FluxLoraTrainer):
    """The same loop on the Krea DiT (candle-gen-krea/src/training.rs:20-160, train_dit.rs:60): adapters on the q / k / v /
    output projections of every block's attention (the gate projection and the modulation table stay frozen); the model
    sees the raw flow time sigma and its raw output is regressed towards eps - x0 (no 1 - sigma, no negation). Items
    hold `latent` [C, h, w] and `txt` [L, layers, text_hidden] (the stacked encoder layers the text fusion consumes).
    The oracle-backend model keeps q / k / v separate, which is what the adapter names address."""
    family, target_suffixes, item_keys = "krea", KREA_TARGETS, ("latent", "txt")

    def __init__(self, cfg, weights: dict[str, torch.Tensor], backend: str = "cpu", device="cpu"):
        from ..models.dit_krea import KreaDiT

        self.cfg, self.backend, self.device = cfg, backend, torch.device("cpu")   # fp32 autograd through the unfused layout
        self.model = KreaDiT(cfg, weights, dtype=torch.float32, device=self.device)
        self.model.w = self.model.bag.w
        for t in self.model.w.values():
            t.requires_grad_(False)

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor("krea_lora_trainer" if self.backend != "cpu" else "cpu_krea_lora_trainer", "krea", self.backend,
                                {"adapters": ["lora", "lokr"], "targets": list(KREA_TARGETS)})

    def loss_on(self, item, t: float, noise: torch.Tensor) -> torch.Tensor:
        x0, eps = item["latent"][None], noise[None]
        xt = (1.0 - t) * x0 + t * eps
        out = self.model.forward_grad(xt, torch.full((1,), t, device=self.device), item["txt"][None])
        return torch.mean((out.float() - (eps - x0)) ** 2)


def krea_trainer_registration(backend: str):
    """`krea_lora_trainer` (kind "trainer"): loads the DiT of a Krea snapshot directory."""
    from ..contracts.gen_core.registry import Registration
    from ..contracts.gen_core.runtime import LoadSpec

    tid = "krea_lora_trainer" if backend != "cpu" else "cpu_krea_lora_trainer"

    def load(spec: LoadSpec) -> KreaLoraTrainer:
        from ..io.safetensors_io import load_dir
        from .krea import KreaPipeline, VARIANTS

        if spec.weights is None or spec.weights.is_file:
            raise InferenceError(f"{tid}: needs a snapshot directory")
        root = Path(spec.weights.path)
        if not (root / "transformer").is_dir():
            raise LoadError(f"{tid}: missing {root / 'transformer'}")
        pipe = KreaPipeline(VARIANTS[0], root, "cpu", torch.device("cpu"))
        return KreaLoraTrainer(pipe.dit_cfg, load_dir(root / "transformer"), backend, "cpu")

    return Registration(descriptor=lambda: SimpleDescriptor(tid, "krea", backend, {"adapters": ["lora", "lokr"]}), load=load)


SDXL_TARGETS = ("attn1.to_q", "attn1.to_k", "attn1.to_v", "attn1.to_out.0", "attn2.to_q", "attn2.to_k", "attn2.to_v",
                "attn2.to_out.0")


class SdxlLoraTrainer(FluxLoraTrainer):
    """The same loop on the SDXL UNet with the noise-prediction objective (candle-gen-sdxl/src/training.rs): adapters on
    the attention projections of every transformer block; the loop's t in (0, 1) picks the DDPM timestep round(999 t),
    x_t = sqrt(a) x0 + sqrt(1 - a) eps with a the cumulative alpha of the scaled-linear table, loss || eps_theta - eps ||^2.
    Items hold `latent` [4, h, w] (scaled VAE latents), `txt` [77, 2048] and `pooled` [1280]; adapter files use the
    `unet.` prefix."""
    family, target_suffixes, item_keys = "sdxl", SDXL_TARGETS, ("latent", "txt", "pooled")

    def __init__(self, cfg, weights: dict[str, torch.Tensor], backend: str = "cpu", device="cpu"):
        from ..contracts.gen_core.sampling.policy import AlphaSchedule
        from ..models.unet_sdxl import SdxlUnet

        self.cfg, self.backend, self.device = cfg, backend, torch.device(device)
        self.model = SdxlUnet(cfg, weights, dtype=torch.float32, device=self.device)
        for t in self.model.w.values():
            t.requires_grad_(False)
        self.alphas = AlphaSchedule.scaled_linear().alphas_cumprod

    def descriptor(self) -> SimpleDescriptor:
        return SimpleDescriptor("sdxl_lora_trainer" if self.backend != "cpu" else "cpu_sdxl_lora_trainer", "sdxl",
                                self.backend, {"adapters": ["lora"], "targets": list(SDXL_TARGETS)})

    def loss_on(self, item, t: float, noise: torch.Tensor) -> torch.Tensor:
        step = min(len(self.alphas) - 1, max(0, round(t * (len(self.alphas) - 1))))
        a = self.alphas[step]
        x0, eps = item["latent"][None], noise[None]
        xt = math.sqrt(a) * x0 + math.sqrt(1.0 - a) * eps
        h, w = x0.shape[2] * 8, x0.shape[3] * 8
        ids = torch.tensor([[h, w, 0, 0, h, w]], dtype=torch.float32, device=self.device)
        out = self.model.forward_grad(xt, torch.full((1,), float(step), device=self.device), item["txt"][None],
                                      item["pooled"][None], ids)
        return torch.mean((out - eps) ** 2)

    def _save(self, path: Path, adapters, c: TrainingConfig, step: int, opt, gen) -> Path:
        out = super()._save(path, adapters, c, step, opt, gen)
        t = load_file(out)                                    # the UNet's adapter files carry the `unet.` prefix
        save_file({k.replace("transformer.", "unet.", 1): v for k, v in t.items()}, out,
                  metadata={"format": "peft-lora", "rank": str(c.rank), "alpha": str(c.alpha), "step": str(step),
                            "base": self.family})
        return out

    def _load_checkpoint(self, path: Path, adapters, opt, gen) -> int:
        t = load_file(path)
        tmp = path.with_name(path.stem + ".resume.safetensors")
        save_file({k.replace("unet.", "transformer.", 1): v for k, v in t.items()}, tmp)
        state = path.with_suffix(".state.safetensors")
        tmp_state = tmp.with_suffix(".state.safetensors")
        tmp_state.write_bytes(state.read_bytes())
        try:
            return super()._load_checkpoint(tmp, adapters, opt, gen)
        finally:
            tmp.unlink(missing_ok=True)
            tmp_state.unlink(missing_ok=True)


def sdxl_trainer_registration(backend: str):
    """`sdxl_lora_trainer` (kind "trainer"): loads the UNet of an SDXL snapshot directory."""
    from ..contracts.gen_core.registry import Registration
    from ..contracts.gen_core.runtime import LoadSpec

    tid = "sdxl_lora_trainer" if backend != "cpu" else "cpu_sdxl_lora_trainer"

    def load(spec: LoadSpec) -> SdxlLoraTrainer:
        from ..io.safetensors_io import load_dir
        from .sdxl import SdxlPipeline

        if spec.weights is None or spec.weights.is_file:
            raise InferenceError(f"{tid}: needs a snapshot directory")
        root = Path(spec.weights.path)
        device = torch.device("cuda", torch.cuda.current_device()) if backend != "cpu" else torch.device("cpu")
        if not (root / "unet").is_dir():
            raise LoadError(f"{tid}: missing {root / 'unet'}")
        pipe = SdxlPipeline(root, "cpu", device)
        return SdxlLoraTrainer(pipe.unet_cfg, load_dir(root / "unet"), backend, device)

    return Registration(descriptor=lambda: SimpleDescriptor(tid, "sdxl", backend, {"adapters": ["lora"]}), load=load)


def trainer_registration(backend: str):
    """`flux1_lora_trainer` (kind "trainer"): loads the DiT of a FLUX snapshot directory and trains adapters on it."""
    from ..contracts.gen_core.registry import Registration
    from ..contracts.gen_core.runtime import LoadSpec

    tid = "flux1_lora_trainer" if backend != "cpu" else "cpu_flux1_lora_trainer"

    def load(spec: LoadSpec) -> FluxLoraTrainer:
        from .flux import FluxPipeline, Variant

        if spec.weights is None or spec.weights.is_file:
            raise InferenceError(f"{tid}: needs a snapshot directory")
        device = torch.device("cuda", torch.cuda.current_device()) if backend != "cpu" else torch.device("cpu")
        pipe = FluxPipeline(Variant.DEV, Path(spec.weights.path), "cpu", device)
        f = Path(spec.weights.path) / Variant.DEV.transformer_file
        if not f.is_file():
            raise LoadError(f"{tid}: missing {f}")
        return FluxLoraTrainer(pipe.dit_cfg, load_file(f), backend, device)

    return Registration(descriptor=lambda: SimpleDescriptor(tid, "flux", backend, {"adapters": ["lora"]}), load=load)
