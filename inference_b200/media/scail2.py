"""SCAIL-2 character animation / motion transfer `scail2_14b` (parity: candle-gen-scail2/src/{pipeline,generate,preprocess,
resize}.rs).

Inputs: a REFERENCE character image, its colour-coded segmentation MASK, and a CONTROL_CLIP carrying the driving video
frames with one colour-coded mask per frame. The colour masks are split into seven binary classes (white, red, green,
blue, yellow, magenta, cyan: a channel counts as on above 225 / 255), average-pooled 8 x 8 to latent resolution and
packed four sub-frames per latent frame (the first frame repeated four times) into 28 channels. The driving clip and its
masks enter at half resolution. The reference image is also read by a CLIP ViT-H/14 tower for image cross-attention.

Long clips are rendered in windows of 81 frames that overlap by 5: the last 5 decoded frames of a window are re-encoded
and pinned (flagged as clean history) at the start of the next, and the overlap is dropped from the later window's
output. `video_mode="replacement"` selects identity replacement (the reference rows are shifted in the rotary table).
Classifier-free guidance 5, flow shift 5, 40 steps; LoRA / LoKr files fold into the DiT weights at load."""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, ConditioningKind, GenerationOutput, GenerationRequest, Generator, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec, ProgressDecoding, ProgressStep
from ..models.dit_scail2 import ClipVisionConfig, Scail2Config, Scail2DiT, ScailClip, random_clip_weights, random_scail2_weights
from ..models.vae_qwen import QwenVaeConfig, WanVaeDecoder, WanVaeEncoder
from .residency import Residency
from .seed import default_seed, seeded_noise_nchw
from .wan import MAX_AREA_14B, TRAIN_TIMESTEPS, FlowUniPc, wan_sigmas

MODEL_ID, FAMILY = "scail2_14b", "scail2"
SEGMENT_LEN, SEGMENT_OVERLAP, DEFAULT_STEPS, DEFAULT_SHIFT, DEFAULT_GUIDANCE, DEFAULT_FPS = 81, 5, 40, 5.0, 5.0, 16
DIM_ALIGN, TEMPORAL_STRIDE, ON_THRESH = 32, 4, (225.0 - 127.5) / 127.5
CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)


def align(v: int) -> int:
    return max(v // DIM_ALIGN, 1) * DIM_ALIGN


def image_to_chw(img: Image, tw: int, th: int, mode: str) -> torch.Tensor:
    """RGB8 -> [3, th, tw] in [-1, 1], resized with `mode` ("bicubic" / "bilinear", pixel centres, no antialiasing)."""
    if len(img.pixels) != img.width * img.height * 3:
        raise InferenceError(f"scail2: image pixel buffer {len(img.pixels)} != {img.width}x{img.height}x3")
    x = torch.frombuffer(bytearray(img.pixels), dtype=torch.uint8).view(img.height, img.width, 3).permute(2, 0, 1).float() / 127.5 - 1.0
    if (img.height, img.width) != (th, tw):
        x = F.interpolate(x[None], size=(th, tw), mode=mode, align_corners=False)[0]
    return x


def downsample_half(x: torch.Tensor) -> torch.Tensor:
    return F.interpolate(x, size=(x.shape[-2] // 2, x.shape[-1] // 2), mode="bilinear", align_corners=False)


def compress_mask_to_latent(mask: torch.Tensor, stride: int = TEMPORAL_STRIDE) -> torch.Tensor:
    """[3, T, H, W] colour mask in [-1, 1] -> [7 * stride, (T - 1) / stride + 1, H / 8, W / 8]."""
    _, T, H, W = mask.shape
    if H % 8 or W % 8:
        raise InferenceError(f"scail2 mask: H,W must be divisible by 8 (got {H}x{W})")
    if stride < 1 or T < 1:
        raise InferenceError("scail2 mask: temporal_stride and T must be >= 1")
    if (T - 1) % stride:
        raise InferenceError(f"scail2 mask: (T-1) must be divisible by temporal_stride (got T={T}, temporal_stride={stride})")
    r, g, b = ((mask[c] > ON_THRESH).float() for c in range(3))
    n = lambda v: 1.0 - v                                                 # noqa: E731
    cls = torch.stack([r * g * b, r * n(g) * n(b), n(r) * g * n(b), n(r) * n(g) * b, r * g * n(b), r * n(g) * b, n(r) * g * b], 1)   # [T, 7, H, W]
    pooled = cls.reshape(T, 7, H // 8, 8, W // 8, 8).mean((3, 5))
    padded = torch.cat([pooled[:1].expand(stride, -1, -1, -1), pooled[1:]], 0)
    return padded.reshape((T - 1) // stride + 1, stride * 7, H // 8, W // 8).permute(1, 0, 2, 3).contiguous()


def vae_align(n: int) -> int:
    return 0 if n == 0 else (n - 1) // TEMPORAL_STRIDE * TEMPORAL_STRIDE + 1


def build_segments(total: int, length: int = SEGMENT_LEN, overlap: int = SEGMENT_OVERLAP) -> list[tuple[int, int]]:
    if total == 0 or length == 0 or overlap >= length:
        return []
    if total <= length:
        return [(0, vae_align(total))]
    segs, start = [], 0
    while start + length <= total:
        segs.append((start, start + length))
        start += length - overlap
    if start < total:
        tail = vae_align(total - start)
        if tail > overlap:
            segs.append((start, start + tail))
    return segs


def apply_clean_history(latent: torch.Tensor, history: torch.Tensor | None) -> torch.Tensor:
    if history is None:
        return latent
    ht = min(history.shape[1], latent.shape[1])
    return latent if ht == 0 else torch.cat([history[:, :ht].to(latent), latent[:, ht:]], 1)


def clip_preprocess(chw: torch.Tensor, size: int) -> torch.Tensor:
    x = F.interpolate(chw[None], size=(size, size), mode="bicubic", align_corners=False) * 0.5 + 0.5
    return (x - torch.tensor(CLIP_MEAN).view(1, 3, 1, 1)) / torch.tensor(CLIP_STD).view(1, 3, 1, 1)


class _Heavy:
    def __init__(self, dit, vae, enc, clip):
        self.dit, self.vae, self.enc, self.clip = dit, vae, enc, clip


class Scail2Pipeline:
    def __init__(self, root: Path, backend: str, device: torch.device, adapters=()):
        self.root, self.backend, self.device, self.adapters = Path(root), backend, device, list(adapters)
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32
        self.raw = json.loads((self.root / "swb_config.json").read_text()) if (self.root / "swb_config.json").exists() else {}
        self.cfg = Scail2Config.from_json(self.raw.get("dit", json.loads((self.root / "config.json").read_text())
                                                       if (self.root / "config.json").exists() else {}))
        self.clip_cfg = ClipVisionConfig(**self.raw["clip"]) if "clip" in self.raw else ClipVisionConfig()
        v = dict(self.raw.get("vae", {}))
        if "dim_mult" in v:
            v["dim_mult"] = tuple(v["dim_mult"])
        self.vae_cfg = QwenVaeConfig(**v)
        self.text_kind = self.raw.get("text", "umt5")

    def load_text(self):
        if self.text_kind == "hash":
            from .wan import HashPromptEncoder

            return HashPromptEncoder(self.cfg.text_dim, self.device, self.dtype)
        from ..models.text_encoders import T5Config, T5Encoder
        from .text_models import T5SentencePieceTokenizer, _load_component
        from .wan import Umt5PromptEncoder

        te, sp = self.root / "text_encoder", self.root / "tokenizer" / "spiece.model"
        if not te.is_dir() or not sp.exists():
            raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks text_encoder/ or tokenizer/spiece.model")
        cfg, w = _load_component(te)
        return Umt5PromptEncoder(T5Encoder(T5Config.from_json(cfg), w, self.device, self.dtype), T5SentencePieceTokenizer(sp))

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir
        from .family import fold_adapters

        for d in ("transformer", "vae", "clip"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks {d}/")
        dit_w = load_dir(self.root / "transformer")
        if self.adapters:
            dit_w = fold_adapters(dit_w, self.adapters, MODEL_ID)
        vae_w = load_dir(self.root / "vae")
        if "encoder.conv_in.weight" not in vae_w:
            raise LoadError(f"{MODEL_ID}: the autoencoder checkpoint has no encoder (reference and driving clips need one)")
        return _Heavy(Scail2DiT(self.cfg, dit_w, self.dtype, self.device), WanVaeDecoder(self.vae_cfg, vae_w, torch.float32, self.device),
                      WanVaeEncoder(self.vae_cfg, vae_w, torch.float32, self.device),
                      ScailClip(self.clip_cfg, load_dir(self.root / "clip"), self.dtype, self.device))

    def encode(self, text, req: GenerationRequest):
        g = req.guidance if req.guidance is not None else DEFAULT_GUIDANCE
        pos = text.encode(req.prompt)[0]
        return pos, (text.encode(req.negative_prompt or "")[0] if g > 1.0 else None)

    @torch.no_grad()
    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress, segment_len=SEGMENT_LEN, overlap=SEGMENT_OVERLAP):
        ref, mask, clip = conditioning_of(req)
        frames, masks = clip.frames, clip.mask_frames
        if not frames:
            raise InferenceError("scail2: a driving video is required")
        if len(masks) != len(frames):
            raise InferenceError(f"scail2: driving_masks ({len(masks)}) must match driving_frames ({len(frames)})")
        tw, th = align(req.width or frames[0].width), align(req.height or frames[0].height)
        steps = req.steps or DEFAULT_STEPS
        guidance = req.guidance if req.guidance is not None else DEFAULT_GUIDANCE
        seed = req.seed if req.seed is not None else default_seed()
        dit, dev = heavy.dit, self.device
        enc = lambda cthw: heavy.enc.encode(cthw[None])[0].float()                       # noqa: E731  [16, T_lat, h, w]
        ref_chw = image_to_chw(ref, tw, th, "bicubic")
        ref_latent = enc(ref_chw[:, None])
        ref_mask28 = compress_mask_to_latent(image_to_chw(mask, tw, th, "bilinear")[:, None]).to(dev)
        lh, lw = ref_latent.shape[2:]
        driving = torch.stack([image_to_chw(f, tw, th, "bicubic") for f in frames])                       # [T, 3, H, W]
        dmask = torch.stack([image_to_chw(m, tw, th, "bilinear") for m in masks], 1)                      # [3, T, H, W]
        pos, neg = cond
        ctx_pos = dit.embed_text(pos)
        ctx_neg = dit.embed_text(neg) if neg is not None else None
        img_ctx = dit.embed_img(heavy.clip.encode(clip_preprocess(ref_chw, self.clip_cfg.image_size)))
        segs = build_segments(len(frames), segment_len, overlap)
        if not segs:
            raise InferenceError(f"scail2: {len(frames)} driving frames leave no window to render")
        sigmas = wan_sigmas(steps, float(req.scheduler_shift) if req.scheduler_shift else DEFAULT_SHIFT)
        pieces, history_px = [], None
        for si, (s0, s1) in enumerate(segs):
            pose_latent = enc(downsample_half(driving[s0:s1]).permute(1, 0, 2, 3))                        # [16, T_lat, h/2, w/2]
            T = pose_latent.shape[1]
            dm28 = compress_mask_to_latent(downsample_half(dmask[:, s0:s1])).to(dev)
            ref_masks = torch.cat([ref_mask28, torch.zeros(28, T, lh, lw, device=dev)], 1)
            hist_lat, hist_mask = None, None
            if history_px is not None:
                hist_lat = enc(history_px)
                ht = min(hist_lat.shape[1], T)
                hist_mask = torch.cat([torch.ones(4, ht, lh, lw, device=dev), torch.zeros(4, T - ht, lh, lw, device=dev)], 1)
            noise = seeded_noise_nchw((seed + si) & ((1 << 64) - 1), 16 * T, lh, lw).reshape(16, T, lh, lw).to(dev).float()
            x = apply_clean_history(noise, hist_lat)
            unipc = FlowUniPc(sigmas) if req.sampler in (None, "unipc", "uni_pc") else None
            for i in range(steps):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{MODEL_ID}: cancelled at step {i} of window {si}")
                xi = apply_clean_history(x, hist_lat)
                t = sigmas[i] * TRAIN_TIMESTEPS
                kw = dict(history_mask=hist_mask, replace_flag=req.video_mode == "replacement")
                v = dit.forward(xi, ref_latent, ref_masks, pose_latent, dm28, ctx_pos, img_ctx, t, **kw)
                if ctx_neg is not None:
                    u = dit.forward(xi, ref_latent, ref_masks, pose_latent, dm28, ctx_neg, img_ctx, t, **kw)
                    v = u + (v - u) * guidance
                x = unipc.step(v[None], x[None], i)[0] if unipc is not None else x + v * (sigmas[i + 1] - sigmas[i])
                x = apply_clean_history(x, hist_lat)
                on_progress(ProgressStep(si * steps + i + 1, steps * len(segs)))
            if si + 1 == len(segs):
                on_progress(ProgressDecoding())
            video = heavy.vae.decode(x[None].float())[0].float().cpu()                                    # [3, T_out, H, W]
            pieces.append(video[:, 0 if si == 0 else overlap:])
            if si + 1 < len(segs):
                history_px = video[:, video.shape[1] - overlap:].contiguous()
        full = torch.cat(pieces, 1)
        u8 = torch.round((full.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 3, 0).contiguous()
        return [Image(width=tw, height=th, pixels=f.numpy().tobytes()) for f in u8]


def conditioning_of(req: GenerationRequest):
    ref = next((c.image for c in req.conditioning if c.kind is ConditioningKind.REFERENCE and c.image is not None), None)
    if ref is None:
        raise InferenceError("scail2: a Reference character image is required")
    mask = next((c.image for c in req.conditioning if c.kind is ConditioningKind.MASK and c.image is not None), None)
    if mask is None:
        raise InferenceError("scail2: a Mask (the reference character's color-coded segmentation mask) is required")
    clip = next((c for c in req.conditioning if c.kind is ConditioningKind.CONTROL_CLIP), None)
    if clip is None:
        raise InferenceError("scail2: a ControlClip (driving video frames + per-frame color masks) is required")
    if not clip.frames:
        raise InferenceError("scail2: the ControlClip has no driving frames")
    return ref, mask, clip


def scail2_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.VIDEO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE, ConditioningKind.MASK, ConditioningKind.CONTROL_CLIP],
            supports_lora=True, supports_lokr=True, samplers=["unipc", "dpm++", "euler"], schedulers=[], supported_guidance_methods=[],
            min_size=32, max_size=1280, max_count=1),
        required_components=[])


class Scail2Generator(Generator):
    def __init__(self, pipe: Scail2Pipeline, descriptor: ModelDescriptor, policy):
        self.pipe, self._descriptor = pipe, descriptor
        sync = torch.cuda.synchronize if pipe.device.type == "cuda" else (lambda: None)
        self.residency = Residency.from_policy(policy, pipe.load_text, pipe.load_heavy, sync)

    def descriptor(self) -> ModelDescriptor:
        return self._descriptor

    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        if any(c.kind is ConditioningKind.MULTI_REFERENCE for c in req.conditioning):
            raise Unsupported(f"{mid}: MultiReference (extra reference characters) is not supported yet - each extra character needs "
                              "its own color-coded segmentation mask; pass exactly one Reference + Mask")
        if req.steps == 0:
            raise InferenceError(f"{mid}: steps must be >= 1 (an explicit 0 renders undenoised noise)")
        if req.width * req.height > MAX_AREA_14B:
            raise InferenceError(f"{mid}: width x height ({req.width}x{req.height}) exceeds the max area {MAX_AREA_14B} px")
        self._descriptor.capabilities.validate_request(mid, req)

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        conditioning_of(req)
        frames = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(video_frames=frames, fps=req.fps or DEFAULT_FPS)


def registration(backend: str = "b200") -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> Scail2Generator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError("scail2: expected a snapshot directory (text_encoder/ transformer/ vae/ clip/ tokenizer/), not a single file")
        if spec.quantize is not None:
            raise Unsupported(f"{mid} does not support on-the-fly Q4/Q8 quantization yet")
        root = Path(spec.weights.path)
        if not root.exists():
            raise LoadError(f"scail2: snapshot dir does not exist: {root}")
        for ad in spec.adapters:
            if ad.kind not in (AdapterKind.LORA, AdapterKind.LOKR):
                raise Unsupported(f"{mid}: adapter kind {ad.kind.value} is not supported")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        return Scail2Generator(Scail2Pipeline(root, backend, device, spec.adapters), scail2_descriptor(backend, prefix), spec.offload_policy)

    return Registration(descriptor=lambda: scail2_descriptor(backend, prefix), load=load)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """Tiny SCAIL-2-shaped snapshot: a 2-layer DiT of width 256 (2 heads of 128), a 3-block CLIP tower on 28 x 28 crops, the
    small z16 autoencoder with its encoder, the weight-free prompt encoder."""
    from ..io.safetensors_io import save_file
    from ..models.vae_qwen import random_wan_vae_encoder_weights, random_wan_vae_weights

    root = Path(root)
    for d in ("transformer", "vae", "clip"):
        (root / d).mkdir(parents=True, exist_ok=True)
    dit = dict(dim=256, ffn_dim=128, num_heads=2, num_layers=2, text_dim=64, text_len=16, clip_dim=32, freq_dim=32)
    clip = dict(image_size=28, patch_size=14, dim=32, num_heads=2, num_layers=3, mlp_dim=64)
    vae = QwenVaeConfig(base_dim=8, dim_mult=(1, 2, 2, 2), num_res_blocks=1)
    save_file(random_scail2_weights(Scail2Config.from_json(dit), seed), root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file(random_clip_weights(ClipVisionConfig(**clip), seed + 1), root / "clip" / "model.safetensors")
    save_file({**random_wan_vae_weights(vae, seed + 2), **random_wan_vae_encoder_weights(vae, seed + 3)}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": dit, "clip": clip, "vae": {"base_dim": vae.base_dim, "dim_mult": list(vae.dim_mult), "num_res_blocks": vae.num_res_blocks},
        "text": "hash"}))
    return root
