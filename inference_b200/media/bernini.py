"""Bernini renderer `bernini_renderer` (parity: candle-gen-bernini/src/{pipeline,config,forward,guidance,preprocess}.rs,
candle-gen-wan/src/rope.rs `apply_source_id` / `assign_source_ids`).

The renderer is the Wan2.2 T2V-A14B network pair (a high-noise and a low-noise expert switched at a timestep boundary)
fine-tuned for packed source conditioning: reference images and conditioning clips are encoded by the video
autoencoder, patch-embedded by the same stem as the noisy target and laid on ONE token axis in front of it, each source
with its own rotary phase (a per-source id added to every rotary lane, ids 1..n, interpolated onto 1..max_trained when
more sources than the training range arrive). Only the target's tokens are read back.

Guidance modes (`video_mode`, or chosen from the conditioning): plain chains of classifier-free differences (`t2v`,
`v2v`, `v2v_chain`, `rv2v`) and adaptive projected guidance in sample space (`t2v_apg`, `v2v_apg`, `r2v_apg`): the
difference of two predicted clean samples is norm-clipped per frame, split along the conditional prediction and its
parallel part damped by eta. On the first low-noise step every guidance weight is scaled once by 0.8.

The heavy lifting is the Wan stack of this package (`WanDiT.forward_tokens`, the z16 autoencoder, UMT5, flow UniPC), so
both backends are served: fp32 oracle on CPU, bf16 on the sm_100a kernels on a CUDA device."""
from __future__ import annotations

import enum
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
from .seed import default_seed, seeded_noise_nchw
from .wan import (MAX_AREA_14B, NEGATIVE_FALLBACK, SIZE_MULTIPLE, TRAIN_TIMESTEPS, FlowUniPc, WanGenerator, WanPipeline,
                  WanVariant, preprocess_i2v_image, wan_sigmas)

MODEL_ID, FAMILY = "bernini_renderer", "bernini"
DEFAULT_STEPS, DEFAULT_FRAMES, DEFAULT_FPS = 40, 81, 16
OMEGA_VID, OMEGA_IMG, OMEGA_TXT, OMEGA_SCALE, ETA, MOMENTUM, NORM_THRESHOLD = 1.25, 4.5, 4.0, 0.8, 0.5, 0.0, 50.0
ROPE_THETA = 10000.0
SAMPLERS = ["uni_pc", "euler", "unipc"]


class Mode(enum.Enum):
    T2V = "t2v"
    T2V_APG = "t2v_apg"
    V2V = "v2v"
    V2V_CHAIN = "v2v_chain"
    V2V_APG = "v2v_apg"
    R2V_APG = "r2v_apg"
    RV2V = "rv2v"

    @property
    def is_apg(self) -> bool:
        return self in (Mode.T2V_APG, Mode.V2V_APG, Mode.R2V_APG)

    @property
    def needs_conditioning(self) -> bool:
        return self not in (Mode.T2V, Mode.T2V_APG)


_TASKS = {"t2i": Mode.T2V_APG, "t2v": Mode.T2V_APG, "i2i": Mode.V2V, "v2v": Mode.V2V_APG, "mv2v": Mode.V2V_APG,
          "ads2v": Mode.V2V_APG, "r2v": Mode.R2V_APG, "rv2v": Mode.RV2V}


def resolve_mode(video_mode: str | None, has_video: bool, has_image: bool) -> Mode:
    """An explicit guidance-mode name wins, then a task name, then the conditioning present."""
    if video_mode:
        for m in Mode:
            if m.value == video_mode:
                return m
        if video_mode in _TASKS:
            return _TASKS[video_mode]
    return {(True, True): Mode.RV2V, (True, False): Mode.V2V_APG, (False, True): Mode.V2V, (False, False): Mode.T2V_APG}[
        (has_video, has_image)]


def check_mode_conditioning(mid: str, mode: Mode, has_source: bool) -> None:
    if mode.needs_conditioning and not has_source:
        raise InferenceError(f"{mid}: guidance mode {mode.value} needs source conditioning (a reference image / video clip) "
                             "but none was provided")
    if not mode.needs_conditioning and has_source:
        raise InferenceError(f"{mid}: guidance mode {mode.value} is text-only but source conditioning was provided (it would "
                             "be silently ignored)")


@dataclass
class BerniniKnobs:
    switch_dit_boundary: float = 0.875
    shift: float = 3.0
    use_src_id_rotary_emb: bool = True
    interpolate_src_id: bool = True
    max_trained_src_id: float = 5.0
    max_sequence_length: int = 512

    @staticmethod
    def from_dir(root: Path) -> "BerniniKnobs":
        f = Path(root) / "bernini_renderer.json"
        if not f.is_file():
            return BerniniKnobs()
        try:
            j = json.loads(f.read_text(encoding="utf-8"))
        except ValueError as e:
            raise LoadError(f"bernini_renderer knobs: parse {f.name} (corrupt snapshot?): {e}") from e
        k = BerniniKnobs()
        for name, typ in (("switch_dit_boundary", float), ("shift", float), ("use_src_id_rotary_emb", bool),
                          ("interpolate_src_id", bool), ("max_trained_src_id", float), ("max_sequence_length", int)):
            if isinstance(j, dict) and isinstance(j.get(name), (int, float, bool)):
                setattr(k, name, typ(j[name]))
        return k


# ---- source ids -------------------------------------------------------------------------------------------------------------
def assign_source_ids(n: int, max_trained: float, interpolate: bool) -> list[float]:
    if n == 0:
        return []
    if interpolate and n > max_trained:
        if n == 1:
            return [1.0]
        step = (max_trained - 1.0) / (n - 1.0)
        return [1.0 + step * i for i in range(n)]
    return [float(i) for i in range(1, n + 1)]


def apply_source_id(cos: torch.Tensor, sin: torch.Tensor, source_id: float, head_dim: int):
    """Adds the phase source_id * theta^(-2k / head_dim) to lane k of the rotary tables [S, head_dim / 2]."""
    if source_id == 0.0:
        return cos, sin
    k = torch.arange(head_dim // 2, dtype=torch.float64)
    ang = source_id * torch.pow(torch.tensor(ROPE_THETA, dtype=torch.float64), -2.0 * k / head_dim)
    ci, si = ang.cos().float().to(cos.device)[None], ang.sin().float().to(cos.device)[None]
    return cos * ci - sin * si, sin * ci + cos * si


class PackedForward:
    """Velocity of the target given sources [(latent, source id)] packed in front of it on the token axis."""

    def __init__(self, knobs: BerniniKnobs):
        self.knobs = knobs
        self._tok: dict = {}

    def _segment(self, dit, lat: torch.Tensor, sid: float, cache: bool):
        key = (id(dit), id(lat))
        if cache and key in self._tok:
            tok, grid = self._tok[key][:2]
        else:
            tok, grid = dit.patch_embed_tokens(lat)
            if cache:
                self._tok[key] = (tok, grid, lat)          # the latent is held so its id stays unique
        cos, sin = dit.grid_rope(grid)
        if self.knobs.use_src_id_rotary_emb:
            cos, sin = apply_source_id(cos, sin, sid, dit.cfg.attention_head_dim)
        return tok, cos, sin, grid

    def velocity(self, dit, target: torch.Tensor, sources, t: float, ctx: torch.Tensor) -> torch.Tensor:
        segs = [self._segment(dit, lat, sid, True) for lat, sid in sources] + [self._segment(dit, target, 0.0, False)]
        grid = segs[-1][3]
        n_target = grid[0] * grid[1] * grid[2]
        x = torch.cat([s[0] for s in segs], dim=1)
        rope = (torch.cat([s[1] for s in segs], 0), torch.cat([s[2] for s in segs], 0))
        out = dit.forward_tokens(x, torch.full((1,), float(t), device=dit.device), ctx, rope)
        _, _, Fr, H, W = target.shape
        return dit.unpatchify(out[:, -n_target:], Fr, H, W).float()

    def combos(self, videos: list[torch.Tensor], images: list[torch.Tensor]) -> dict[str, list]:
        k = self.knobs
        vi_ids = assign_source_ids(len(videos) + len(images), k.max_trained_src_id, k.interpolate_src_id)
        i_ids = assign_source_ids(len(images), k.max_trained_src_id, k.interpolate_src_id)
        v = [(x, vi_ids[n]) for n, x in enumerate(videos)]
        return {"none": [], "v": v, "i": [(x, i_ids[n]) for n, x in enumerate(images)],
                "vi": v + [(x, vi_ids[len(videos) + n]) for n, x in enumerate(images)]}


# ---- adaptive projected guidance (per frame: reductions over channel, row, column of [B, C, T, H, W]) --------------------------
APG_DIMS = (1, 3, 4)


class MomentumBuffer:
    def __init__(self, momentum: float):
        self.momentum, self.running = momentum, None

    def update(self, diff: torch.Tensor) -> torch.Tensor:
        self.running = diff if self.running is None else diff + self.momentum * self.running
        return self.running


def _normalize_diff(diff, base, buf: MomentumBuffer | None, eta: float, norm_threshold: float):
    if buf is not None:
        diff = buf.update(diff)
    if norm_threshold > 0.0:
        n = diff.pow(2).sum(APG_DIMS, keepdim=True).sqrt()
        diff = diff * (norm_threshold / n).clamp(max=1.0)
    v1 = base / base.pow(2).sum(APG_DIMS, keepdim=True).sqrt().clamp(min=1e-12)
    par = (diff * v1).sum(APG_DIMS, keepdim=True) * v1
    return (diff - par) + eta * par


def normalized_guidance(cond, uncond, scale: float, buf: MomentumBuffer | None, eta: float, norm_threshold: float):
    """uncond + scale * [orthogonal + eta * parallel] of the (momentum-averaged, norm-clipped) difference cond - uncond,
    split along cond. eta = 1 with no clipping is plain classifier-free guidance."""
    return uncond + scale * _normalize_diff(cond - uncond, cond, buf, eta, norm_threshold)


def normalized_guidance_chain(uncond, preds, scales, bufs, eta: float, norm_thresholds):
    if not (len(preds) == len(scales) == len(bufs) == len(norm_thresholds)):
        raise InferenceError(f"normalized_guidance_chain: preds={len(preds)} but scales={len(scales)} bufs={len(bufs)} "
                             f"norm_thresholds={len(norm_thresholds)} (all must match)")
    out = uncond
    for i, cond in enumerate(preds):
        prev = uncond if i == 0 else preds[i - 1]
        out = out + scales[i] * _normalize_diff(cond - prev, cond, bufs[i], eta, norm_thresholds[i])
    return out


def num_momentum_buffers(mode: Mode) -> int:
    return {Mode.T2V_APG: 1, Mode.V2V_APG: 1, Mode.R2V_APG: 2}.get(mode, 0)


@dataclass
class GuidanceParams:
    omega_vid: float = OMEGA_VID
    omega_img: float = OMEGA_IMG
    omega_txt: float = OMEGA_TXT
    eta: float = ETA
    norm_threshold: tuple[float, float] = (NORM_THRESHOLD, NORM_THRESHOLD)


def guided_velocity(pf: PackedForward, mode: Mode, dit, noisy, videos, images, t: float, sigma: float, ctx_cond, ctx_uncond,
                    g: GuidanceParams, bufs: list[MomentumBuffer]) -> torch.Tensor:
    c = pf.combos(videos, images)
    v = lambda src, cond: pf.velocity(dit, noisy, c[src], t, ctx_cond if cond else ctx_uncond)        # noqa: E731
    nz = noisy.float()

    def chain(*terms):
        acc = terms[0][0]
        for (cur, w), (prev, _) in zip(terms[1:], terms[:-1]):
            acc = acc + (cur - prev) * w
        return acc

    to_x = lambda vel: nz - sigma * vel                           # noqa: E731
    from_x = lambda x: (nz - x) / sigma                           # noqa: E731
    if mode is Mode.T2V:
        return chain((v("none", False), 0.0), (v("none", True), g.omega_txt))
    if mode is Mode.V2V:
        return chain((v("vi", False), 0.0), (v("vi", True), g.omega_txt))
    if mode is Mode.V2V_CHAIN:
        return chain((v("none", False), 0.0), (v("v", False), g.omega_vid), (v("vi", True), g.omega_txt))
    if mode is Mode.RV2V:
        return chain((v("none", False), 0.0), (v("v", False), g.omega_vid), (v("vi", False), g.omega_img), (v("vi", True), g.omega_txt))
    if mode in (Mode.T2V_APG, Mode.V2V_APG):
        src = "none" if mode is Mode.T2V_APG else "vi"
        x0, xt = to_x(v(src, False)), to_x(v(src, True))
        return from_x(normalized_guidance(xt, x0, g.omega_txt, bufs[0], g.eta, g.norm_threshold[0]))
    x0, xi, xti = to_x(v("none", False)), to_x(v("i", False)), to_x(v("i", True))
    return from_x(normalized_guidance_chain(x0, [xi, xti], [g.omega_img, g.omega_txt], bufs, g.eta, list(g.norm_threshold)))


# ---- generator ------------------------------------------------------------------------------------------------------------
def _sources(req: GenerationRequest) -> tuple[list[list[Image]], list[Image]]:
    clips, images = [], []
    for c in req.conditioning:
        if c.kind is ConditioningKind.REFERENCE and c.image is not None:
            images.append(c.image)
        elif c.kind is ConditioningKind.MULTI_REFERENCE:
            images.extend(c.images)
        elif c.kind is ConditioningKind.VIDEO_CLIP:
            clips.append(c.frames)
    return clips, images


class BerniniPipeline(WanPipeline):
    def __init__(self, root: Path, backend: str, device: torch.device):
        self.knobs = BerniniKnobs.from_dir(root)
        super().__init__(root, backend, device, WanVariant(MODEL_ID, self.knobs.switch_dit_boundary, self.knobs.shift,
                                                           OMEGA_TXT, OMEGA_TXT))

    def load_heavy(self):
        from ..models.vae_qwen import WanVaeEncoder, random_wan_vae_encoder_weights

        heavy = super().load_heavy()
        if self.random_init is not None and self.backend == "b200":
            heavy.encoder = WanVaeEncoder(self.vae_cfg, random_wan_vae_encoder_weights(self.vae_cfg, int(self.random_init) + 3),
                                          torch.float32, self.device)
        else:
            from ..io.safetensors_io import load_dir

            vae_w = load_dir(self.root / "vae")
            if "encoder.conv_in.weight" in vae_w:
                heavy.encoder = WanVaeEncoder(self.vae_cfg, vae_w, torch.float32, self.device)
        return heavy

    def encode(self, text, req: GenerationRequest):
        return text.encode(req.prompt), text.encode(req.negative_prompt or NEGATIVE_FALLBACK)

    def encode_image(self, heavy, img: Image, req) -> torch.Tensor:
        return heavy.encoder.encode(preprocess_i2v_image(img, req.width, req.height)).to(self.device, self.dtype)

    def encode_clip(self, heavy, frames: list[Image], req) -> torch.Tensor:
        if not frames:
            raise InferenceError(f"{MODEL_ID}: empty conditioning video clip")
        if len(frames) % 4 != 1:
            raise InferenceError(f"{MODEL_ID}: video-clip frame count must be 1 + 4k (got {len(frames)})")
        clip = torch.cat([preprocess_i2v_image(f, req.width, req.height) for f in frames], dim=2)
        return heavy.encoder.encode(clip).to(self.device, self.dtype)

    @torch.no_grad()
    def render(self, heavy, cond, req: GenerationRequest, on_progress) -> list[list[Image]]:
        steps = req.steps or DEFAULT_STEPS
        frames = req.frames or DEFAULT_FRAMES
        seed = req.seed if req.seed is not None else default_seed()
        dev, dt = self.device, self.dtype
        clips, images = _sources(req)
        mode = resolve_mode(req.video_mode, bool(clips), bool(images))
        if (clips or images) and heavy.encoder is None:
            raise LoadError(f"{MODEL_ID}: the autoencoder checkpoint has no encoder (source conditioning needs one)")
        vids = [self.encode_clip(heavy, c, req) for c in clips]
        imgs = [self.encode_image(heavy, i, req) for i in images]
        pos, neg = cond
        ctx = {id(m): (m.embed_text(pos), m.embed_text(neg)) for m in (heavy.high, heavy.low)}
        lt, lh, lw = (frames - 1) // 4 + 1, req.height // 8, req.width // 8
        C = self.dit_cfg.out_channels
        x = seeded_noise_nchw(seed, C * lt, lh, lw).reshape(1, C, lt, lh, lw).to(dev).float()
        shift = float(req.scheduler_shift) if req.scheduler_shift else self.knobs.shift
        sigmas = wan_sigmas(steps, shift)
        unipc = FlowUniPc(sigmas) if req.sampler in (None, "uni_pc", "unipc") else None
        pf = PackedForward(self.knobs)
        bufs = [MomentumBuffer(MOMENTUM) for _ in range(num_momentum_buffers(mode))]
        g = GuidanceParams(omega_txt=req.guidance if req.guidance is not None else OMEGA_TXT)
        boundary, switched = self.knobs.switch_dit_boundary * TRAIN_TIMESTEPS, False
        for i in range(steps):
            if req.cancel.is_cancelled():
                raise Canceled(f"{MODEL_ID}: cancelled at step {i}")
            t = sigmas[i] * TRAIN_TIMESTEPS
            dit = heavy.high if t >= boundary else heavy.low
            if t < boundary and not switched:                     # once, on the first low-noise step
                switched = True
                g.omega_txt, g.omega_vid, g.omega_img = g.omega_txt * OMEGA_SCALE, g.omega_vid * OMEGA_SCALE, g.omega_img * OMEGA_SCALE
            vel = guided_velocity(pf, mode, dit, x.to(dt), vids, imgs, t, sigmas[i], *ctx[id(dit)], g, bufs)
            x = unipc.step(vel, x, i) if unipc is not None else x + vel * (sigmas[i + 1] - sigmas[i])
            on_progress(ProgressStep(i + 1, steps))
        on_progress(ProgressDecoding())
        video = heavy.vae.decode(x.float())[0].float()
        u8 = torch.round((video.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).permute(1, 2, 3, 0).contiguous().cpu()
        return [[Image(width=req.width, height=req.height, pixels=f.numpy().tobytes()) for f in u8[:frames]]]


def bernini_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family=FAMILY, backend=backend, modality=Modality.VIDEO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False,
            conditioning=[ConditioningKind.REFERENCE, ConditioningKind.MULTI_REFERENCE, ConditioningKind.VIDEO_CLIP],
            supports_lora=False, supports_lokr=False, samplers=list(SAMPLERS), schedulers=[], supported_guidance_methods=[],
            min_size=16, max_size=1280, max_count=1, supports_sequential_offload=True),
        required_components=[])


class BerniniRenderer(WanGenerator):
    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt:
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.frames != 1 and req.width * req.height > MAX_AREA_14B:
            raise InferenceError(f"{mid}: width x height ({req.width}x{req.height}) exceeds the max area {MAX_AREA_14B} px")
        if req.frames is not None and (req.frames < 1 or req.frames % 4 != 1):
            raise InferenceError(f"{mid}: num_frames must be 1 + 4k (got {req.frames})")
        clips, images = _sources(req)
        check_mode_conditioning(mid, resolve_mode(req.video_mode, bool(clips), bool(images)), bool(clips or images))

    def generate(self, req: GenerationRequest, on_progress=lambda p: None) -> GenerationOutput:
        self.validate(req)
        videos = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        if (req.frames or DEFAULT_FRAMES) == 1:
            return GenerationOutput(images=videos[0][:1])
        return GenerationOutput(video_frames=videos[0], fps=req.fps or DEFAULT_FPS)


def registration(backend: str = "b200") -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> BerniniRenderer:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise LoadError(f"{mid}: expected a snapshot directory (text_encoder/ transformer/ transformer_2/ vae/ tokenizer/), "
                            "not a single file")
        reject_unknown_components(spec.components, [], mid)
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid} does not support control / VACE / IP-adapter overlays")
        if spec.adapters:
            raise Unsupported(f"{mid} does not support LoRA/LoKr adapters")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        return BerniniRenderer(BerniniPipeline(Path(spec.weights.path), backend, device), bernini_descriptor(backend, prefix),
                               spec.offload_policy)

    return Registration(descriptor=lambda: bernini_descriptor(backend, prefix), load=load)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """The tiny two-expert Wan snapshot (16-channel stem) plus the autoencoder's encoder and a knobs sidecar."""
    from ..io.safetensors_io import load_file, save_file
    from ..models.vae_qwen import QwenVaeConfig, random_wan_vae_encoder_weights
    from .wan import write_synthetic_snapshot as wan_snapshot

    root = wan_snapshot(root, seed)
    raw = json.loads((root / "swb_config.json").read_text())
    v = dict(raw["vae"])
    v["dim_mult"] = tuple(v["dim_mult"])
    f = root / "vae" / "diffusion_pytorch_model.safetensors"
    w = load_file(f)
    w.update({k: t.bfloat16() for k, t in random_wan_vae_encoder_weights(QwenVaeConfig(**v), seed + 3).items()})
    save_file(w, f)
    (root / "bernini_renderer.json").write_text(json.dumps({"switch_dit_boundary": 0.875, "shift": 3.0}))
    return root
