"""Shared provider scaffolding for flow-matching image / video families.

Every diffusion family of the reference is the same outer program around a different network (the reference repeats
it per crate: `candle-gen-*/src/pipeline.rs` + `lib.rs`): read a snapshot, encode the prompt (and the negative prompt
when classifier-free guidance is on), draw seeded CPU noise, integrate a sigma table with the shared solver framework
while calling the denoiser once or twice per evaluation, decode latents to RGB8, report progress, honour
cancellation and the offload policy. `FamilyPipeline` is that program; a family subclasses it with its network, its
sigma table, its conditioning and its guidance rule, and `family_registrations` turns variants into registry entries
for both bundles (`<id>` on the sm_100a backend, `cpu_<id>` on the fp32 oracle backend).

Snapshot conventions shared by all families built on this module: `swb_config.json` in the snapshot root may carry
`{"text": "hash"}` (weight-free prompt encoder for synthetic snapshots), `{"random_init": seed}` (build random
weights on the device, read no files; benchmarks) and per-component dimension overrides.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator,
                                            Modality, ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import (SCHEDULERS, SOLVERS, FlowModelSampling, TorchLatentOps, denoise, get_solver,
                                           schedule_sigmas)
from ..contracts.gen_core.traits import reject_unknown_components
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw


@dataclass
class Variant:
    """One registered model id of a family."""
    id: str
    family: str
    default_steps: int
    default_guidance: float | None = None      # None: guidance-distilled / CFG-free (negative prompts rejected)
    modality: Modality = Modality.IMAGE
    conditioning: tuple[ConditioningKind, ...] = ()
    min_size: int = 256
    max_size: int = 2048
    size_multiple: int = 16
    supports_lora: bool = False
    supports_lokr: bool = False
    embedded_guidance: bool = False             # the guidance scale is an input of the network (one forward per step)
    fixed_sampler: bool = False                 # the model has its own sampler: no sampler / scheduler menu
    max_count: int = 8
    extra: dict = field(default_factory=dict)   # family-specific constants (checkpoint file names, shifts, ...)

    @property
    def uses_cfg(self) -> bool:
        return self.default_guidance is not None and not self.embedded_guidance


def rgb8_image(img: torch.Tensor, width: int, height: int) -> Image:
    """[3, H, W] in [-1, 1] (any float dtype / device) -> host RGB8, round-half-even like the reference's
    `round_rgb8` (candle-gen/src/lib.rs:188-280)."""
    host = torch.round((img.float().clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 0).contiguous().cpu()
    return Image(width=width, height=height, pixels=host.numpy().tobytes())


def video_frames_rgb8(video: torch.Tensor, width: int, height: int) -> list[Image]:
    """[3, F, H, W] in [-1, 1] -> one host RGB8 image per frame (round-half-even)."""
    u8 = torch.round((video.float().clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()
    return [Image(width=width, height=height, pixels=f.numpy().tobytes()) for f in u8]


class FamilyPipeline:
    """Paths and configuration only; components are built by the residency owner when first needed.

    Subclass hooks: `load_text`, `load_heavy`, `native_sigmas`, `encode`, `velocity`, `decode`; optional
    `combine` (guidance rule), `latent_shape`, `time_of` (what the network is conditioned on for a sigma)."""

    latent_channels = 16
    latent_downscale = 8
    pid_space: str | None = None       # the PiD latent space of this family's VAE: `use_pid` then decodes through media/pid.py

    def __init__(self, variant: Variant, root: Path, backend: str, device: torch.device):
        self.variant, self.root, self.backend, self.device = variant, Path(root), backend, device
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32
        self.raw: dict = {}
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            self.raw = json.loads(cfg_path.read_text())
        self.text_kind = self.raw.get("text", "model")
        self.random_init = self.raw.get("random_init")
        self.adapters: list = []
        self.pid_spec: tuple[Path, Path] | None = None        # (PiD checkpoint file, Gemma-2 snapshot directory)
        self._pid_engine = None
        self.timings: dict | None = None      # set to a dict to collect device-timed "step_ms" / "decode_ms"

    def pid_engine(self, use_pid: bool):
        """The super-resolving pixel decoder of this family's latent space, loaded by the first request that asks."""
        if not use_pid or self.pid_spec is None or self.pid_space is None:
            return None
        if self._pid_engine is None:
            from .pid import PidEngine

            self._pid_engine = PidEngine.load(self.pid_spec[0], self.pid_spec[1], self.pid_space, self.backend)
        return self._pid_engine

    # ---- hooks ---------------------------------------------------------------------------------------------------
    def load_text(self):
        raise NotImplementedError

    def load_heavy(self):
        raise NotImplementedError

    def native_sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        raise NotImplementedError

    def encode(self, text, req: GenerationRequest):
        """-> (positive conditioning, negative conditioning or None)."""
        g = self.guidance(req)
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or "") if self.cfg_active(g) else None
        return pos, neg

    def velocity(self, heavy, x: torch.Tensor, sigma: float, cond) -> torch.Tensor:
        """One network evaluation: the flow velocity dx / d sigma at (x, sigma) for one conditioning."""
        raise NotImplementedError

    def decode(self, heavy, z: torch.Tensor, req: GenerationRequest) -> list[Image]:
        raise NotImplementedError

    def cfg_active(self, guidance: float | None) -> bool:
        return self.variant.uses_cfg and guidance is not None and guidance > 1.0

    def combine(self, cond_v: torch.Tensor, uncond_v: torch.Tensor, guidance: float) -> torch.Tensor:
        return uncond_v + (cond_v - uncond_v) * guidance

    def output_fps(self, req: GenerationRequest) -> int | None:
        return req.fps

    def step_guidance(self, step: int, steps: int, guidance: float) -> float:
        """Guidance scale of evaluation `step` (0-based) out of `steps`; constant unless a family schedules it."""
        return guidance

    def latent_shape(self, req: GenerationRequest) -> tuple[int, int, int]:
        return self.latent_channels, req.height // self.latent_downscale, req.width // self.latent_downscale

    def scheduler_mu(self, req: GenerationRequest) -> float:
        return req.scheduler_shift or 0.0

    # ---- shared program ------------------------------------------------------------------------------------------
    def guidance(self, req: GenerationRequest) -> float | None:
        if self.variant.default_guidance is None:
            return None
        g = req.true_cfg if req.true_cfg is not None else req.guidance
        return float(g) if g is not None else self.variant.default_guidance

    def sigmas(self, steps: int, req: GenerationRequest) -> list[float]:
        if req.scheduler is None:
            return self.native_sigmas(steps, req)
        return schedule_sigmas(req.scheduler, FlowModelSampling(mu=self.scheduler_mu(req)), steps)

    def initial_latent(self, seed: int, req: GenerationRequest) -> torch.Tensor:
        c, h, w = self.latent_shape(req)
        return seeded_noise_nchw(seed, c, h, w)

    def render(self, heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        guidance = self.guidance(req)
        pos, neg = cond
        base_seed = req.seed if req.seed is not None else default_seed()
        dev, dt = self.device, self.dtype
        sigmas = self.sigmas(steps, req)
        solver, ops, ms = get_solver(req.sampler or "euler"), TorchLatentOps(), FlowModelSampling()
        events = [] if (self.timings is not None and dev.type == "cuda") else None
        pid = self.pid_engine(req.use_pid)
        if req.use_pid:
            from .pid import check_pid_request, resolve_pid_decoder

            check_pid_request(pid, req, v.id)     # no engine / capture not wired / over budget: refused before any step

        def one_image(seed: int):
            if events is not None:
                events.clear()
            x = self.initial_latent(seed, req).to(dev, dt).contiguous()
            state = {"step": 0}

            def run_model(x_in, sigma):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{v.id}: cancelled at step {state['step']}")
                if events is not None:
                    events.append((torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)))
                    events[-1][0].record()
                vel = self.velocity(heavy, x_in, float(sigma), pos).float()
                if neg is not None:
                    vel = self.combine(vel, self.velocity(heavy, x_in, float(sigma), neg).float(),
                                       self.step_guidance(state["step"], steps, guidance))
                if events is not None:
                    events[-1][1].record()
                state["step"] += 1
                if state["step"] <= steps:
                    on_progress(ProgressStep(state["step"], steps))
                return vel.to(dt).contiguous()

            x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:            # solvers that skip the final evaluation at sigma 0
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{v.id}: cancelled before decode")
            on_progress(ProgressDecoding())
            if events is not None:
                d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                d0.record()
            if pid is not None:          # the latent the VAE would get; the image comes back `scale` x larger
                px = resolve_pid_decoder(pid, req, seed, v.id).decode(x.float().cpu())
                out = [rgb8_image(px[0], px.shape[3], px.shape[2])]
            else:
                out = self.decode(heavy, x.float(), req)
            if events is not None:
                d1.record()
                torch.cuda.synchronize()
                self.timings["step_ms"] = [a.elapsed_time(b) for a, b in events]
                self.timings["decode_ms"] = d0.elapsed_time(d1)
            return out

        per_seed = for_each_image_seed(base_seed, req.count, one_image)
        return [img for imgs in per_seed for img in imgs]


class FamilyGenerator(Generator):
    def __init__(self, pipe: FamilyPipeline, descriptor: ModelDescriptor, policy: OffloadPolicy | None):
        self.pipe, self._descriptor = pipe, descriptor
        sync = torch.cuda.synchronize if pipe.device.type == "cuda" else (lambda: None)
        self.residency = Residency.from_policy(policy, pipe.load_text, pipe.load_heavy, sync)

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid, v = self._descriptor.id, self.pipe.variant
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt and not v.extra.get("promptless"):
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.steps == 0:
            raise InferenceError(f"{mid}: steps must be >= 1 (an explicit 0 renders undenoised noise)")
        if req.width % v.size_multiple or req.height % v.size_multiple:
            raise InferenceError(f"{mid}: width/height must be multiples of {v.size_multiple} "
                                 f"(got {req.width}x{req.height})")
        hook = getattr(self.pipe, "validate", None)
        if hook is not None:
            hook(req)

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        if self.pipe.variant.modality is Modality.VIDEO:
            return GenerationOutput(video_frames=images, fps=self.pipe.output_fps(req))
        return GenerationOutput(images=images)


def family_descriptor(v: Variant, backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + v.id, family=v.family, backend=backend, modality=v.modality,
        capabilities=Capabilities(
            supports_negative_prompt=v.uses_cfg and not v.extra.get("no_negative"), supports_guidance=v.default_guidance is not None,
            supports_true_cfg=v.uses_cfg,
            conditioning=list(v.conditioning), supports_lora=v.supports_lora, supports_lokr=v.supports_lokr,
            samplers=[] if v.fixed_sampler else list(v.extra.get("samplers", SOLVERS)), schedulers=[] if v.fixed_sampler else list(SCHEDULERS),
            supported_guidance_methods=[], min_size=v.min_size,
            max_size=v.max_size, max_count=v.max_count, supports_sequential_offload=True),
        required_components=[])


def family_registrations(variants: list[Variant], pipeline_cls: Callable[..., FamilyPipeline], backend: str = "b200"
                         ) -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"

    def loader(v: Variant):
        def load(spec: LoadSpec) -> FamilyGenerator:
            mid = prefix + v.id
            if spec.weights is None or spec.weights.is_file:
                raise Unsupported(f"{mid}: needs a snapshot directory")
            if spec.quantize is not None and not v.extra.get("quants"):
                raise Unsupported(f"{mid}: quantised loading ({spec.quantize.name}) is not supported")
            has_pid = getattr(pipeline_cls, "pid_space", None) is not None
            reject_unknown_components(spec.components, ["pid_gemma"] if has_pid else [], mid)
            pid_spec = None
            if spec.pid is not None or "pid_gemma" in spec.components:
                if not has_pid:
                    raise Unsupported(f"{mid}: no pixel decoder exists for this family's latent space")
                if spec.pid is None or not spec.pid.is_file or "pid_gemma" not in spec.components or spec.components["pid_gemma"].is_file:
                    raise LoadError(f"{mid}: the pixel decoder needs LoadSpec.pid (the converted checkpoint file) and the "
                                    "'pid_gemma' component (a Gemma-2 snapshot directory)")
                pid_spec = (Path(spec.pid.path), Path(spec.components["pid_gemma"].path))
            if spec.control or spec.extra_controls or spec.ip_adapter:
                raise Unsupported(f"{mid}: control branches and IP adapters are not supported by this provider")
            for ad in spec.adapters:
                ok = (ad.kind is AdapterKind.LORA and v.supports_lora) or (ad.kind is AdapterKind.LOKR and v.supports_lokr)
                if not ok:
                    raise Unsupported(f"{mid}: adapter kind {ad.kind.value} is not supported")
            if backend == "b200":
                if not torch.cuda.is_available():
                    raise LoadError(f"{mid}: no CUDA device")
                device = torch.device("cuda", torch.cuda.current_device())
            else:
                device = torch.device("cpu")
            pipe = pipeline_cls(v, Path(spec.weights.path), backend, device)
            pipe.adapters = list(spec.adapters)
            pipe.pid_spec = pid_spec
            pipe.quantize = spec.quantize
            return FamilyGenerator(pipe, family_descriptor(v, backend, prefix), spec.offload_policy)
        return load

    return [Registration(descriptor=(lambda v=v: family_descriptor(v, backend, prefix)), load=loader(v)) for v in variants]


class HashPromptEncoder:
    """Weight-free stand-in for a family's prompt encoder (synthetic snapshots, benchmarks): deterministic
    pseudo-random features of the prompt bytes, [1, L, dim] (and a pooled [1, pooled_dim] vector when asked)."""

    def __init__(self, dim: int, device, dtype, pooled_dim: int = 8, min_len: int = 8, layers: int = 0):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(dim * max(1, layers), pooled_dim, device, dtype)
        self.min_len, self.layers, self.dim = min_len, layers, dim

    def encode(self, prompt: str, length: int | None = None):
        n = length if length is not None else self.min_len + len(prompt.encode("utf-8"))
        c = self.h.encode(prompt, n)
        if self.layers:
            c.txt = c.txt.view(1, n, self.layers, self.dim)
        return c


def merged_adapters(weights: dict[str, torch.Tensor], adapters: list, mid: str) -> dict[str, torch.Tensor]:
    """Low-rank adapter files merged into a state dict at load (LoRA only)."""
    from ..io.safetensors_io import load_file
    from .train import merge_lora

    for ad in adapters:
        if not Path(ad.path).is_file():
            raise LoadError(f"{mid}: adapter file {ad.path} not found")
        weights = merge_lora(weights, load_file(ad.path), ad.scale if ad.scale is not None else 1.0)
    return weights


def load_vl_text_tower(mid: str, root: Path, device, deepest_layer: int):
    """(CausalLmTextEncoder, tokenizer) for families conditioned on intermediate layers of a Qwen3-VL language tower
    stored under `text_encoder/` (+ `tokenizer/tokenizer.json`): the vision tower is dropped and decoder layers above
    `deepest_layer` are never run."""
    import tokenizers

    from ..io.safetensors_io import load_dir
    from ..models.qwen3_vl import language_model_config
    from ..models.text_encoders import CausalLmTextEncoder

    te, tk = Path(root) / "text_encoder", Path(root) / "tokenizer" / "tokenizer.json"
    if not te.is_dir() or not tk.exists():
        raise LoadError(f"{mid}: snapshot {root} lacks text_encoder/ or tokenizer/tokenizer.json")
    cfg = language_model_config(json.loads((te / "config.json").read_text()))
    w = {}
    for k, v in load_dir(te).items():
        for pre in ("model.language_model.", "language_model.model.", "language_model."):
            if k.startswith(pre):
                w["model." + k[len(pre):]] = v
                break
        else:
            if k.startswith("model.") and not k.startswith("model.visual"):
                w[k] = v
    enc = CausalLmTextEncoder(cfg, w, device, skip_last=max(0, cfg.num_layers - deepest_layer))
    return enc, tokenizers.Tokenizer.from_file(str(tk))


ADAPTER_ROOTS = ("", "model.diffusion_model.", "diffusion_model.", "transformer.", "net.", "model.", "lora_unet_", "lycoris_")


def fold_adapters(weights: dict[str, torch.Tensor], adapters: list, mid: str) -> dict[str, torch.Tensor]:
    """LoRA and LoKr adapter files folded into a state dict at load, stacked in order. A module is addressed by its
    dotted path under any of the usual roots, or by the kohya spelling (dots replaced by underscores); a target that
    matches no 2-D weight of the model is an error, never a silent partial application."""
    from ..io.safetensors_io import load_file
    from .adapters import parse_thirdparty

    out = dict(weights)
    modules = {k[: -len(".weight")] for k, v in out.items() if k.endswith(".weight") and v.dim() == 2}
    flat = {m.replace(".", "_"): m for m in modules}

    def route(name: str) -> str:
        for root in ADAPTER_ROOTS:
            if name.startswith(root):
                n = name[len(root):]
                hit = n if n in modules else flat.get(n.replace(".", "_"))
                if hit is not None:
                    return hit
        raise LoadError(f"{mid}: adapter targets '{name}', which the model does not have")

    for ad in adapters:
        if not Path(ad.path).is_file():
            raise LoadError(f"{mid}: adapter file {ad.path} not found")
        t = load_file(ad.path)
        user = ad.scale if ad.scale is not None else 1.0
        if ad.kind is AdapterKind.LOKR:
            lokr, loha = parse_thirdparty(t)
            if not lokr and not loha:
                raise LoadError(f"{mid}: {ad.path} holds no LoKr / LoHa factors")
            for mod, f in {**lokr, **loha}.items():
                key = route(mod) + ".weight"
                w = out[key]
                out[key] = (w.float() + f.delta(tuple(w.shape), user).to(w.device)).to(w.dtype)
            continue
        pairs: dict[str, dict] = {}
        for k, v in t.items():
            for leaf, slot in ((".lora_A.weight", "a"), (".lora_down.weight", "a"), (".lora_B.weight", "b"),
                               (".lora_up.weight", "b"), (".alpha", "alpha")):
                if k.endswith(leaf):
                    pairs.setdefault(k[: -len(leaf)], {})[slot] = v
        if not pairs:
            raise LoadError(f"{mid}: {ad.path} holds no LoRA factors")
        for mod, f in pairs.items():
            if "a" not in f or "b" not in f:
                raise LoadError(f"{mid}: adapter module '{mod}' lacks a down or an up factor")
            key = route(mod) + ".weight"
            a, b, w = f["a"].float(), f["b"].float(), out[key]
            r = a.shape[0]
            alpha = float(f["alpha"].flatten()[0]) if "alpha" in f else float(r)
            out[key] = (w.float() + (b @ a).to(w.device) * (user * alpha / r)).to(w.dtype)
    return out
