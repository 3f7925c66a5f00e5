"""Wan 2.2 A14B video providers `wan2_2_t2v_14b` (text -> video) and `wan2_2_i2v_14b` (image -> video), and their
`cpu_*` twins on the fp32 backend (parity: candle-gen-wan/src/wan14b.rs, pipeline.rs, scheduler.rs, text_encode.rs,
config.rs).

generate(): UMT5 encodes the prompt (512 positions; rows past the prompt's length are zeroed) -> flow-matching steps
over `sigma = shift * s / (1 + (shift - 1) * s)`, s from 1 to 1 / 1000, shift 12 -> at every step the high-noise expert
(timestep >= 875) or the low-noise expert predicts the velocity with classifier-free guidance (4.0 / 3.0) ->
the 16-channel video autoencoder turns (frames - 1) / 4 + 1 latent frames into `frames` RGB frames (default 81 frames,
16 fps, 40 steps). The default integrator is the model's own second-order multistep predictor-corrector (`FlowUniPc`,
also selected by `uni_pc`); any other sampler name routes to the shared solver framework (`euler`, ...).

`wan2_2_i2v_14b` differs in its conditioning and constants: the Reference image (cover-fit bilinear resize, centre crop)
becomes frame 0 of an otherwise zero clip, the autoencoder's encoder turns that clip into 16-channel latents, a
4-channel mask marks latent frame 0, and the 20 channels are concatenated to the 16 noise channels of every network
input (36 in, 16 out); expert boundary 0.900, shift 5, guidance 3.5 / 3.5.

Snapshot layout (diffusers): `transformer/` (high-noise expert), `transformer_2/` (low-noise expert; optional for
single-network checkpoints), `text_encoder/` + `tokenizer/`, `vae/`; `swb_config.json` overrides dimensions for synthetic
snapshots."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator,
                                            Modality, ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import SOLVERS, FlowModelSampling, TorchLatentOps, denoise, get_solver
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_wan import WanConfig, WanDiT
from ..models.vae_qwen import QwenVaeConfig, WanVaeDecoder, WanVaeEncoder
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw

MODEL_ID = "wan2_2_t2v_14b"
DEFAULT_STEPS, DEFAULT_FRAMES, DEFAULT_FPS = 40, 81, 16
BOUNDARY, FLOW_SHIFT, GUIDANCE_HIGH, GUIDANCE_LOW = 0.875, 12.0, 4.0, 3.0
TRAIN_TIMESTEPS, TEXT_TOKENS, SIZE_MULTIPLE = 1000, 512, 16
MAX_AREA_14B = 1280 * 720


@dataclass(frozen=True)
class WanVariant:
    id: str
    boundary: float
    shift: float
    guidance_high: float
    guidance_low: float
    i2v: bool = False
    stride: int = 8             # spatial compression of the autoencoder (16 for the z48 autoencoder of the 5B model)
    fps: int = DEFAULT_FPS


T2V_14B = WanVariant(MODEL_ID, BOUNDARY, FLOW_SHIFT, GUIDANCE_HIGH, GUIDANCE_LOW)
I2V_14B = WanVariant("wan2_2_i2v_14b", 0.900, 5.0, 3.5, 3.5, i2v=True)
WAN_VARIANTS = (T2V_14B, I2V_14B)


def i2v_reference(req: GenerationRequest) -> Image | None:
    for c in req.conditioning:
        if c.kind is ConditioningKind.REFERENCE and c.image is not None:
            return c.image
    return None


def preprocess_i2v_image(img: Image, width: int, height: int) -> torch.Tensor:
    """Cover-fit bilinear resize (pixel centres, clamped), centre crop -> [1, 3, 1, height, width] in [-1, 1]."""
    import torch.nn.functional as F

    if len(img.pixels) != img.width * img.height * 3:
        raise InferenceError(f"i2v image buffer {len(img.pixels)} != {img.width}x{img.height}x3")
    scale = max(width / img.width, height / img.height)
    nw, nh = max(round(img.width * scale), width), max(round(img.height * scale), height)
    x = torch.frombuffer(bytearray(img.pixels), dtype=torch.uint8).view(img.height, img.width, 3).permute(2, 0, 1)[None].double()
    y = F.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False)
    x1, y1 = (nw - width) // 2, (nh - height) // 2
    return (y[:, :, y1:y1 + height, x1:x1 + width] / 255.0 * 2.0 - 1.0).float()[:, :, None]
NEGATIVE_FALLBACK = ("色调艳丽，过曝，静态，细节模糊不清，字幕，风格，作品，画作，画面，静止，整体发灰，最差质量，低质量，JPEG压缩残留，丑陋的，残缺的，"
                     "多余的手指，画得不好的手部，画得不好的脸部，畸形的，毁容的，形态畸形的肢体，手指融合，静止不动的画面，杂乱的背景，三条腿，背景人很多，倒着走")


def wan_sigmas(steps: int, shift: float = FLOW_SHIFT) -> list[float]:
    n = max(1, steps)
    ramp = [1.0 + (1.0 / TRAIN_TIMESTEPS - 1.0) * i / n for i in range(n)]            # linspace(1, 1/N, n + 1)[:-1]
    out = [shift * s / (1.0 + (shift - 1.0) * s) for s in ramp]
    out[0] -= 1e-6
    return out + [0.0]


class FlowUniPc:
    """Second-order multistep predictor-corrector for flow matching (the checkpoint's default integrator: UniPC with
    the B(h) = e^h - 1 variant, data prediction, lower order on the first and the last step;
    candle-gen-wan/src/scheduler.rs:101-213). It works in half-log-SNR lambda = log((1 - sigma) / sigma): with
    h = lambda_t - lambda_s, a step from sigma_s to sigma_t is
    x_t = (sigma_t / sigma_s) x_s - (1 - sigma_t)(e^{-h} - 1)(x0_s + correction), where the correction extrapolates the
    data prediction from the previous step (predictor) and, once the model has been evaluated at x_t, also interpolates
    towards the new prediction (corrector, applied at the start of the next step)."""

    def __init__(self, sigmas: list[float], order: int = 2):
        self.sigmas, self.order = sigmas, order
        self.steps = len(sigmas) - 1
        self.history: list[torch.Tensor] = []         # data predictions of the last evaluated points, newest last
        self.last_sample: torch.Tensor | None = None
        self.last_order, self.warm = 1, 0

    @staticmethod
    def _lam(sigma: float) -> float:
        import math

        return math.inf if sigma <= 0.0 else math.log((1.0 - sigma) / sigma)

    def _base(self, x, m0, s_from: float, s_to: float):
        import math

        h = self._lam(s_to) - self._lam(s_from)
        em1 = math.expm1(-h)                              # e^{-h} - 1 (-1 at the terminal sigma 0)
        return x * (s_to / s_from) - m0 * ((1.0 - s_to) * em1), h, em1

    def _predict(self, x, i: int, order: int):
        m0 = self.history[-1]
        xt, h, em1 = self._base(x, m0, self.sigmas[i], self.sigmas[i + 1])
        if order >= 2 and len(self.history) >= 2:
            rk = (self._lam(self.sigmas[i - 1]) - self._lam(self.sigmas[i])) / h
            xt = xt - (self.history[-2] - m0) * ((1.0 - self.sigmas[i + 1]) * em1 * 0.5 / rk)
        return xt

    def _correct(self, x0_new, i: int, order: int):
        """Re-does the step i-1 -> i from the stored sample, now knowing the data prediction at its end point."""
        m0 = self.history[-1]                              # prediction at sigma_{i-1}
        s_from, s_to = self.sigmas[i - 1], self.sigmas[i]
        xt, h, em1 = self._base(self.last_sample, m0, s_from, s_to)
        a_t, d_new = 1.0 - s_to, x0_new - m0
        if order == 1 or len(self.history) < 2:
            return xt - d_new * (a_t * em1 * 0.5)
        hh = -h
        rk = (self._lam(self.sigmas[i - 2]) - self._lam(s_from)) / h
        phi1 = em1 / hh - 1.0
        b0, b1 = phi1 / em1, (phi1 / hh - 0.5) * 2.0 / em1
        r0, r1 = (b0 - b1) / (1.0 - rk), (b1 - rk * b0) / (1.0 - rk)
        return xt - ((self.history[-2] - m0) * (r0 / rk) + d_new * r1) * (a_t * em1)

    def step(self, velocity: torch.Tensor, x: torch.Tensor, i: int) -> torch.Tensor:
        """x at sigma_i and the model's velocity there -> x at sigma_{i+1}."""
        x0 = x - velocity * self.sigmas[i]
        if i > 0 and self.last_sample is not None:
            x = self._correct(x0, i, self.last_order)
        self.history = (self.history + [x0])[-2:]
        order = min(self.order, self.steps - i, self.warm + 1)
        self.last_sample, self.last_order = x, order
        self.warm = min(self.warm + 1, self.order)
        return self._predict(x, i, order)


class Umt5PromptEncoder:
    def __init__(self, t5, tokenizer, tokens: int = TEXT_TOKENS):
        self.t5, self.tok, self.tokens = t5, tokenizer, tokens

    def encode(self, prompt: str) -> torch.Tensor:
        """[1, tokens, d_model]: the encoder's states for the prompt's tokens, zeros after them."""
        ids = (self.tok.sp.encode(prompt) + [self.tok.eos])[: self.tokens]
        n = len(ids)
        padded = torch.tensor([ids + [self.tok.pad] * (self.tokens - n)], dtype=torch.int64)
        mask = torch.tensor([[1] * n + [0] * (self.tokens - n)])
        out = self.t5.encode(padded, mask).clone()
        out[:, n:] = 0
        return out


class HashPromptEncoder:
    def __init__(self, dim: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(dim, 8, device, dtype)

    def encode(self, prompt: str) -> torch.Tensor:
        return self.h.encode(prompt, 16).txt


@dataclass
class _Heavy:
    high: Any
    low: Any
    vae: Any
    encoder: Any = None


class WanPipeline:
    def __init__(self, root: Path, backend: str, device: torch.device, variant: WanVariant = T2V_14B):
        self.root, self.backend, self.device, self.variant = Path(root), backend, device, variant
        self.dit_cfg, self.vae_cfg, self.text_kind, self.random_init = WanConfig(), QwenVaeConfig(), "umt5", None
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                self.dit_cfg = WanConfig.from_json(raw["dit"])
            if "vae" in raw:
                v = dict(raw["vae"])
                if "dim_mult" in v:
                    v["dim_mult"] = tuple(v["dim_mult"])
                self.vae_cfg = QwenVaeConfig(**v)
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = WanConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32
        if variant.i2v and self.dit_cfg.in_channels == self.dit_cfg.out_channels:
            import dataclasses

            self.dit_cfg = dataclasses.replace(self.dit_cfg, in_channels=self.dit_cfg.out_channels + 4 + self.vae_cfg.z_dim)

    def load_text(self):
        if self.text_kind == "hash":
            return HashPromptEncoder(self.dit_cfg.text_dim, self.device, self.dtype)
        from ..models.text_encoders import T5Config, T5Encoder
        from .text_models import T5SentencePieceTokenizer, _load_component

        te, sp = self.root / "text_encoder", self.root / "tokenizer" / "spiece.model"
        if not te.is_dir() or not sp.exists():
            raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks text_encoder/ or tokenizer/spiece.model")
        cfg, w = _load_component(te)
        return Umt5PromptEncoder(T5Encoder(T5Config.from_json(cfg), w, self.device, self.dtype), T5SentencePieceTokenizer(sp))

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir
        from ..models.dit_wan import random_wan_weights
        from ..models.vae_qwen import random_wan_vae_weights

        if self.random_init is not None and self.backend == "b200":
            seed = int(self.random_init)
            mk = lambda s: WanDiT(self.dit_cfg, random_wan_weights(self.dit_cfg, s, 0.02, torch.bfloat16, self.device),      # noqa: E731
                                  self.dtype, self.device)
            enc = None
            if self.variant.i2v:
                from ..models.vae_qwen import random_wan_vae_encoder_weights

                enc = WanVaeEncoder(self.vae_cfg, random_wan_vae_encoder_weights(self.vae_cfg, seed + 3), torch.float32, self.device)
            return _Heavy(mk(seed), mk(seed + 1), WanVaeDecoder(self.vae_cfg, random_wan_vae_weights(self.vae_cfg, seed + 2),
                                                                torch.float32, self.device), enc)
        for d in ("transformer", "vae"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{self.variant.id}: snapshot {self.root} lacks {d}/")
        high = WanDiT(self.dit_cfg, load_dir(self.root / "transformer"), self.dtype, self.device)
        low = high
        if (self.root / "transformer_2").is_dir():
            low = WanDiT(self.dit_cfg, load_dir(self.root / "transformer_2"), self.dtype, self.device)
        vae_w = load_dir(self.root / "vae")
        enc = WanVaeEncoder(self.vae_cfg, vae_w, torch.float32, self.device) if self.variant.i2v else None
        if enc is not None and "encoder.conv_in.weight" not in enc.w:
            raise LoadError(f"{self.variant.id}: the autoencoder checkpoint has no encoder (image -> video needs one)")
        return _Heavy(high, low, WanVaeDecoder(self.vae_cfg, vae_w, torch.float32, self.device), enc)

    def encode(self, text, req: GenerationRequest):
        g = req.guidance
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or NEGATIVE_FALLBACK) if g is None or g > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[list[Image]]:
        steps = req.steps or DEFAULT_STEPS
        frames = req.frames or DEFAULT_FRAMES
        base_seed = req.seed if req.seed is not None else default_seed()
        var = self.variant
        lt, lh, lw = (frames - 1) // 4 + 1, req.height // var.stride, req.width // var.stride
        dev, dt = self.device, self.dtype
        sigmas = wan_sigmas(steps, float(req.scheduler_shift) if req.scheduler_shift else var.shift)
        y = None
        if var.i2v:
            ref = i2v_reference(req)
            if ref is None:
                raise InferenceError(f"{var.id}: image -> video requires a Reference image")
            clip = torch.zeros(1, 3, frames, req.height, req.width)
            clip[:, :, :1] = preprocess_i2v_image(ref, req.width, req.height)
            z_video = heavy.encoder.encode(clip)                                              # [1, 16, lt, lh, lw]
            mask = torch.zeros(1, 4, *z_video.shape[2:], device=z_video.device)
            mask[:, :, 0] = 1.0
            y = torch.cat([mask, z_video], dim=1).to(dev, dt)
        native_unipc = req.sampler in (None, "uni_pc", "unipc")        # the model's own multistep integrator
        solver, ops, ms = get_solver(req.sampler or "euler"), TorchLatentOps(), FlowModelSampling()
        conds = [c for c in cond if c is not None]
        # the text projection does not depend on the step: once per expert and prompt
        ctx = {id(m): [m.embed_text(c) for c in conds] for m in {id(heavy.high): heavy.high, id(heavy.low): heavy.low}.values()}
        C = self.dit_cfg.out_channels

        def one_video(seed: int) -> list[Image]:
            x = seeded_noise_nchw(seed, C * lt, lh, lw).reshape(1, C, lt, lh, lw).to(dev, dt).contiguous()
            state = {"step": 0}

            def run_model(x_in, sigma):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{var.id}: cancelled at step {state['step']}")
                t = float(sigma) * TRAIN_TIMESTEPS
                high = t >= var.boundary * TRAIN_TIMESTEPS
                model = heavy.high if high else heavy.low
                g = req.guidance if req.guidance is not None else (var.guidance_high if high else var.guidance_low)
                tt = torch.full((1,), t, device=dev)
                if y is not None:
                    x_in = torch.cat([x_in, y], dim=1)
                outs = [model.forward(x_in, tt, c, embedded=True).float() for c in ctx[id(model)]]
                vel = outs[0] if len(outs) == 1 else outs[1] + (outs[0] - outs[1]) * g
                state["step"] += 1
                if state["step"] <= steps:
                    on_progress(ProgressStep(state["step"], steps))
                return vel.to(dt).contiguous()

            if native_unipc:
                stepper, xf = FlowUniPc(sigmas), x.float()
                for i in range(steps):
                    xf = stepper.step(run_model(xf.to(dt).contiguous(), sigmas[i]).float(), xf, i)
                x = xf
            else:
                x = solver.sample(ops, ms, lambda xx, s: denoise(ops, ms, xx, s, run_model), x, sigmas, seed)
            while state["step"] < steps:
                state["step"] += 1
                on_progress(ProgressStep(state["step"], steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{var.id}: cancelled before decode")
            on_progress(ProgressDecoding())
            video = heavy.vae.decode(x.float())[0].float()                              # [3, F, H, W]
            u8 = torch.round((video.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()
            return [Image(width=req.width, height=req.height, pixels=f.numpy().tobytes()) for f in u8[:frames]]

        return for_each_image_seed(base_seed, req.count, one_video)


def wan_descriptor(backend: str, prefix: str = "", variant: WanVariant = T2V_14B) -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + variant.id, family="wan", backend=backend, modality=Modality.VIDEO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE] if variant.i2v else [],
            supports_lora=False, supports_lokr=False, samplers=list(SOLVERS), schedulers=[],
            supported_guidance_methods=[], min_size=256, max_size=1280, max_count=1, supports_sequential_offload=True),
        required_components=[])


class WanGenerator(Generator):
    def __init__(self, pipe: WanPipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
        self.pipe, self._descriptor = pipe, descriptor
        sync = torch.cuda.synchronize if pipe.backend == "b200" else (lambda: None)
        self.residency = Residency.from_policy(policy, pipe.load_text, pipe.load_heavy, sync)

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt:
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.frames is not None and (req.frames < 1 or (req.frames - 1) % 4):
            raise InferenceError(f"{mid}: frames must be 4k + 1 (got {req.frames})")
        if req.width * req.height > MAX_AREA_14B:
            raise InferenceError(f"{mid}: {req.width}x{req.height} exceeds the {MAX_AREA_14B}-pixel frame budget")
        if self.pipe.variant.i2v and i2v_reference(req) is None:
            raise InferenceError(f"{mid}: image -> video requires a Reference image")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        videos = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(video_frames=videos[0], fps=req.fps or self.pipe.variant.fps)


def _load(backend: str, prefix: str, variant: WanVariant = T2V_14B) -> Callable[[LoadSpec], WanGenerator]:
    def load(spec: LoadSpec) -> WanGenerator:
        mid = prefix + variant.id
        if spec.weights is None or spec.weights.is_file:
            raise Unsupported(f"{mid}: needs a snapshot directory")
        if spec.quantize is not None:
            raise Unsupported(f"{mid}: quantised loading ({spec.quantize.name}) is not supported")
        reject_unknown_components(spec.components, [], mid)
        if spec.control or spec.extra_controls or spec.ip_adapter or spec.adapters:
            raise Unsupported(f"{mid}: adapters, control branches and IP adapters are not supported by this provider")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        return WanGenerator(WanPipeline(Path(spec.weights.path), backend, device, variant),
                            wan_descriptor(backend, prefix, variant), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=(lambda v=v: wan_descriptor(backend, prefix, v)), load=_load(backend, prefix, v))
            for v in WAN_VARIANTS]


def write_synthetic_snapshot(root, seed: int = 0, i2v: bool = False) -> Path:
    """A tiny random two-expert snapshot in the diffusers directory layout with the weight-free prompt encoder;
    `i2v` widens the patch embedding to 36 channels and adds the autoencoder's encoder."""
    from ..io.safetensors_io import save_file
    from ..models.dit_wan import random_wan_weights
    from ..models.vae_qwen import random_wan_vae_encoder_weights, random_wan_vae_weights

    root = Path(root)
    dit = WanConfig(num_attention_heads=2, attention_head_dim=128, num_layers=2, ffn_dim=256, text_dim=64,
                    in_channels=36 if i2v else 16)
    vae = QwenVaeConfig(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    for name, s in (("transformer", seed), ("transformer_2", seed + 1)):
        (root / name).mkdir(parents=True, exist_ok=True)
        save_file({k: v.bfloat16() for k, v in random_wan_weights(dit, s).items()},
                  root / name / "diffusion_pytorch_model.safetensors")
    (root / "vae").mkdir(exist_ok=True)
    vae_w = random_wan_vae_weights(vae, seed + 2)
    if i2v:
        vae_w.update(random_wan_vae_encoder_weights(vae, seed + 3))
    save_file({k: v.bfloat16() for k, v in vae_w.items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {"num_attention_heads": 2, "attention_head_dim": 128, "num_layers": 2, "ffn_dim": 256, "text_dim": 64,
                "in_channels": dit.in_channels},
        "vae": {"base_dim": vae.base_dim, "dim_mult": list(vae.dim_mult), "num_res_blocks": vae.num_res_blocks},
        "text": "hash"}))
    return root
