"""Wan-VACE controllable video `wan_vace` (Wan2.1-VACE-14B) (parity: candle-gen-wan/src/{vace,model_vace}.rs, config.rs).

Mode-agnostic at the engine boundary: the caller builds a control clip and a per-frame mask (person replacement: the
clip with the person region neutralised + the person mask; extension / bridging: the kept frames + a mask over the span
to generate) and passes them as one CONTROL_CLIP conditioning. The clip is split by the binarised mask into an
"inactive" (kept) and a "reactive" (to be regenerated) video, both encoded by the z16 autoencoder (32 channels); the
mask itself is unfolded 8 x 8 into 64 channels at latent resolution and resampled in time; together they are the
96-channel control latent. REFERENCE images become extra leading latent frames (with zero reactive half and zero mask)
that are dropped from the result.

The network is the Wan 14B DiT plus a control branch: eight extra blocks run on the control tokens (the first adds the
embedded noisy tokens to its projected input); each emits a hint through its own projection, and hint j is added, times
`control_scale`, to the main stream after block `vace_layers[j]`. Classifier-free guidance 5, flow shift 5, 50 UniPC
steps, 16 fps. The Wan stack of this package serves both backends."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, ProgressDecoding, ProgressStep
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_wan import WanConfig, WanDiT, random_wan_weights
from .seed import default_seed, seeded_noise_nchw
from .wan import (MAX_AREA_14B, NEGATIVE_FALLBACK, SIZE_MULTIPLE, TRAIN_TIMESTEPS, FlowUniPc, WanGenerator, WanPipeline, WanVariant,
                  preprocess_i2v_image, wan_sigmas)

MODEL_ID = "wan_vace"
DEFAULT_STEPS, DEFAULT_GUIDANCE, FLOW_SHIFT, DEFAULT_FPS = 50, 5.0, 5.0, 16
VAE_T, VAE_S = 4, 8
VACE_LAYERS_14B, VACE_IN_CHANNELS = (0, 5, 10, 15, 20, 25, 30, 35), 96


class WanVaceDiT(WanDiT):
    def __init__(self, cfg: WanConfig, weights, vace_layers, dtype=torch.float32, device="cpu"):
        super().__init__(cfg, weights, dtype, device)
        self.vace_layers = tuple(vace_layers)
        self.w["vace_patch_embedding.weight"] = self.w["vace_patch_embedding.weight"].reshape(cfg.dim, -1).contiguous()

    def embed_control(self, control: torch.Tensor, n_tokens: int) -> torch.Tensor:
        """Control latent [B, 96, F, H, W] -> tokens [B, n_tokens, dim] (zero rows appended when shorter)."""
        emb = self._lin(self.patchify(control.to(self.device, self.dtype)), "vace_patch_embedding")
        if emb.shape[1] > n_tokens:
            raise InferenceError(f"wan-vace: control token count {emb.shape[1]} exceeds latent token count {n_tokens}; the "
                                 "control clip resolution must match the generation resolution")
        return torch.nn.functional.pad(emb, (0, 0, 0, n_tokens - emb.shape[1]))

    @torch.no_grad()
    def forward_vace(self, z, timestep, control_emb, ctx, scales) -> torch.Tensor:
        if len(scales) != len(self.vace_layers):
            raise InferenceError(f"wan-vace: control scales len {len(scales)} != vace_layers len {len(self.vace_layers)}")
        _, _, Fr, H, W = z.shape
        x, grid = self.patch_embed_tokens(z)
        rope = self.grid_rope(grid)
        _, tproj = self._time(timestep, x.shape[0])
        hints, c = {}, control_emb
        for j, layer in enumerate(self.vace_layers):
            p = f"vace_blocks.{j}"
            if j == 0:
                c = self._lin(c, p + ".proj_in") + x
            c = self._block(c, p, tproj, ctx, rope)
            hints[layer] = self._lin(c, p + ".proj_out").float() * float(scales[j])
        return self.unpatchify(self.forward_tokens(x, timestep, ctx, rope, hints), Fr, H, W)


def binarize_mask(mask: torch.Tensor) -> torch.Tensor:
    return (mask > 0.5).float()


def nearest_exact_temporal(x: torch.Tensor, axis: int, out_t: int) -> torch.Tensor:
    f = x.shape[axis]
    idx = [min(max(int(((i + 0.5) * f / out_t) // 1), 0), f - 1) for i in range(out_t)]
    return x.index_select(axis, torch.tensor(idx, device=x.device))


def prepare_masks(mask: torch.Tensor, patch: int, num_ref: int) -> torch.Tensor:
    """[1, C, F, H, W] in [0, 1] -> [1, 64, ceil(F / 4) + num_ref, H / 8, W / 8]: channel 0 unfolded 8 x 8 into channels,
    frames resampled nearest-exact, zero frames in front for the references."""
    _, _, f, h, w = mask.shape
    nh, nw = h // (VAE_S * patch) * patch, w // (VAE_S * patch) * patch
    m = mask[0, 0, :, :nh * VAE_S, :nw * VAE_S].reshape(f, nh, VAE_S, nw, VAE_S).permute(2, 4, 0, 1, 3).reshape(VAE_S * VAE_S, f, nh, nw)
    m = nearest_exact_temporal(m, 1, -(-f // VAE_T))
    if num_ref:
        m = torch.cat([torch.zeros(VAE_S * VAE_S, num_ref, nh, nw, device=m.device), m], 1)
    return m[None]


def prepare_video_latents(encode, video: torch.Tensor, mask: torch.Tensor, references) -> torch.Tensor:
    m = binarize_mask(mask)
    lat = torch.cat([encode(video * (1.0 - m)), encode(video * m)], 1)
    for r in references:
        rl = encode(r)
        lat = torch.cat([torch.cat([rl, torch.zeros_like(rl)], 1), lat], 2)
    return lat


def control_clip(req: GenerationRequest):
    for c in req.conditioning:
        if c.kind is ConditioningKind.CONTROL_CLIP:
            return c
    return None


class WanVacePipeline(WanPipeline):
    def __init__(self, root: Path, backend: str, device: torch.device):
        super().__init__(root, backend, device, WanVariant(MODEL_ID, 0.0, FLOW_SHIFT, DEFAULT_GUIDANCE, DEFAULT_GUIDANCE))
        raw = {}
        if (self.root / "swb_config.json").exists():
            raw = json.loads((self.root / "swb_config.json").read_text())
        elif (self.root / "transformer" / "config.json").exists():
            raw = json.loads((self.root / "transformer" / "config.json").read_text())
        self.vace_layers = tuple(raw.get("vace_layers", VACE_LAYERS_14B))

    def load_heavy(self):
        from ..io.safetensors_io import load_dir
        from ..models.vae_qwen import (WanVaeDecoder, WanVaeEncoder, random_wan_vae_encoder_weights, random_wan_vae_weights)
        from .wan import _Heavy

        if self.random_init is not None and self.backend == "b200":
            seed = int(self.random_init)
            dit_w = random_vace_weights(self.dit_cfg, self.vace_layers, seed, 0.02)
            vae_w = {**random_wan_vae_weights(self.vae_cfg, seed + 2), **random_wan_vae_encoder_weights(self.vae_cfg, seed + 3)}
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks {d}/")
            dit_w, vae_w = load_dir(self.root / "transformer"), load_dir(self.root / "vae")
            if "vace_patch_embedding.weight" not in dit_w:
                raise LoadError(f"{MODEL_ID}: transformer/ has no control branch (vace_patch_embedding / vace_blocks)")
            if "encoder.conv_in.weight" not in vae_w:
                raise LoadError(f"{MODEL_ID}: the autoencoder checkpoint has no encoder (the control clip needs one)")
        dit = WanVaceDiT(self.dit_cfg, dit_w, self.vace_layers, self.dtype, self.device)
        return _Heavy(dit, dit, WanVaeDecoder(self.vae_cfg, vae_w, torch.float32, self.device),
                      WanVaeEncoder(self.vae_cfg, vae_w, torch.float32, self.device))

    def _clip_tensor(self, frames: list[Image], req) -> torch.Tensor:
        if not frames:
            raise InferenceError("wan-vace: control clip has no frames")
        return torch.cat([preprocess_i2v_image(f, req.width, req.height) for f in frames], 2)

    @torch.no_grad()
    def render(self, heavy, cond, req: GenerationRequest, on_progress) -> list[list[Image]]:
        clip = control_clip(req)
        if clip is None:
            raise InferenceError("wan-vace: requires a ControlClip")
        steps = req.steps or DEFAULT_STEPS
        guidance = req.guidance if req.guidance is not None else DEFAULT_GUIDANCE
        seed = req.seed if req.seed is not None else default_seed()
        dev, dt, dit = self.device, self.dtype, heavy.high
        video = self._clip_tensor(clip.frames, req)
        mask = (self._clip_tensor(clip.mask_frames, req) + 1.0) * 0.5
        if mask.shape[2] != video.shape[2]:
            raise InferenceError(f"wan-vace: {video.shape[2]} control frames but {mask.shape[2]} mask frames")
        refs = [preprocess_i2v_image(c.image, req.width, req.height) for c in req.conditioning
                if c.kind is ConditioningKind.REFERENCE and c.image is not None]
        encode = lambda v: heavy.encoder.encode(v).float().cpu()                    # noqa: E731
        control = torch.cat([prepare_video_latents(encode, video, mask, refs),
                             prepare_masks(mask, self.dit_cfg.patch_size[1], len(refs))], 1)
        _, _, T, lh, lw = control.shape
        pt, ph, pw = self.dit_cfg.patch_size
        control_emb = dit.embed_control(control, (T // pt) * (lh // ph) * (lw // pw))
        pos, neg = cond
        ctx_pos = dit.embed_text(pos)
        ctx_neg = dit.embed_text(neg) if (neg is not None and guidance > 1.0) else None
        scales = [req.control_scale if getattr(req, "control_scale", None) is not None else 1.0] * len(dit.vace_layers)
        C = self.dit_cfg.out_channels
        x = seeded_noise_nchw(seed, C * T, lh, lw).reshape(1, C, T, lh, lw).to(dev).float()
        sigmas = wan_sigmas(steps, float(req.scheduler_shift) if req.scheduler_shift else FLOW_SHIFT)
        unipc = FlowUniPc(sigmas) if req.sampler in (None, "uni_pc", "unipc") else None
        for i in range(steps):
            if req.cancel.is_cancelled():
                raise Canceled(f"{MODEL_ID}: cancelled at step {i}")
            t = torch.full((1,), sigmas[i] * TRAIN_TIMESTEPS, device=dev)
            v = dit.forward_vace(x.to(dt), t, control_emb, ctx_pos, scales).float()
            if ctx_neg is not None:
                u = dit.forward_vace(x.to(dt), t, control_emb, ctx_neg, scales).float()
                v = u + (v - u) * guidance
            x = unipc.step(v, x, i) if unipc is not None else x + v * (sigmas[i + 1] - sigmas[i])
            on_progress(ProgressStep(i + 1, steps))
        on_progress(ProgressDecoding())
        video_out = heavy.vae.decode(x[:, :, len(refs):].float())[0].float()
        u8 = torch.round((video_out.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()
        return [[Image(width=req.width, height=req.height, pixels=f.numpy().tobytes()) for f in u8[:len(clip.frames)]]]


def vace_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="wan", backend=backend, modality=Modality.VIDEO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False,
            conditioning=[ConditioningKind.CONTROL_CLIP, ConditioningKind.REFERENCE], supports_lora=False, supports_lokr=False,
            samplers=["uni_pc", "euler", "unipc"], schedulers=[], supported_guidance_methods=[], min_size=256, max_size=1280,
            max_count=1, supports_sequential_offload=True),
        required_components=[])


class WanVaceGenerator(WanGenerator):
    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt:
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.width * req.height > MAX_AREA_14B:
            raise InferenceError(f"{mid}: {req.width}x{req.height} exceeds the {MAX_AREA_14B}-pixel frame budget")
        clip = control_clip(req)
        if clip is None:
            raise InferenceError(f"{mid}: requires a ControlClip (control frames + per-frame masks)")
        if not clip.frames or (len(clip.frames) - 1) % 4:
            raise InferenceError(f"{mid}: the control clip must have 4k + 1 frames (got {len(clip.frames)})")
        if len(clip.mask_frames) != len(clip.frames):
            raise InferenceError(f"{mid}: {len(clip.frames)} control frames but {len(clip.mask_frames)} mask frames")

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        videos = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(video_frames=videos[0], fps=req.fps or DEFAULT_FPS)


def registration(backend: str = "b200") -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> WanVaceGenerator:
        mid = prefix + MODEL_ID
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
        return WanVaceGenerator(WanVacePipeline(Path(spec.weights.path), backend, device), vace_descriptor(backend, prefix),
                                spec.offload_policy)

    return Registration(descriptor=lambda: vace_descriptor(backend, prefix), load=load)


def random_vace_weights(cfg: WanConfig, vace_layers, seed: int = 0, std: float = 0.05, in_channels: int = VACE_IN_CHANNELS):
    w = random_wan_weights(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 77)
    pt, ph, pw = cfg.patch_size
    w["vace_patch_embedding.weight"] = torch.randn(cfg.dim, in_channels, pt, ph, pw, generator=g) * std
    w["vace_patch_embedding.bias"] = torch.randn(cfg.dim, generator=g) * 0.01
    for j in range(len(vace_layers)):
        for k, v in list(w.items()):
            if k.startswith("blocks.0."):
                w[f"vace_blocks.{j}." + k[len("blocks.0."):]] = torch.randn(v.shape, generator=g) * (std if v.dim() > 1 else 0.02) + \
                    (1.0 if k.endswith("norm_q.weight") or k.endswith("norm_k.weight") or k.endswith("norm2.weight") else 0.0)
        if j == 0:
            w["vace_blocks.0.proj_in.weight"], w["vace_blocks.0.proj_in.bias"] = torch.randn(cfg.dim, cfg.dim, generator=g) * std, torch.zeros(cfg.dim)
        w[f"vace_blocks.{j}.proj_out.weight"] = torch.randn(cfg.dim, cfg.dim, generator=g) * std
        w[f"vace_blocks.{j}.proj_out.bias"] = torch.zeros(cfg.dim)
    return w


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """The tiny Wan snapshot with a one-layer control branch after block 0 and the autoencoder's encoder."""
    from ..io.safetensors_io import load_file, save_file
    from ..models.vae_qwen import QwenVaeConfig, random_wan_vae_encoder_weights
    from .wan import write_synthetic_snapshot as wan_snapshot

    root = wan_snapshot(root, seed)
    raw = json.loads((root / "swb_config.json").read_text())
    cfg = WanConfig.from_json(raw["dit"])
    f = root / "transformer" / "diffusion_pytorch_model.safetensors"
    base = load_file(f)
    extra = {k: v for k, v in random_vace_weights(cfg, (0,), seed + 5).items() if k.startswith("vace_")}
    save_file({**base, **{k: v.bfloat16() for k, v in extra.items()}}, f)
    v = dict(raw["vae"])
    v["dim_mult"] = tuple(v["dim_mult"])
    vf = root / "vae" / "diffusion_pytorch_model.safetensors"
    vw = load_file(vf)
    vw.update({k: t.bfloat16() for k, t in random_wan_vae_encoder_weights(QwenVaeConfig(**v), seed + 3).items()})
    save_file(vw, vf)
    raw["vace_layers"] = [0]
    (root / "swb_config.json").write_text(json.dumps(raw))
    return root
