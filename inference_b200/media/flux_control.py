"""FLUX.1-dev with a ControlNet branch (pose / canny / depth maps): a bespoke provider driven by name, like PuLID.

The control branch (Shakker-Labs FLUX.1-dev-ControlNet-Union-Pro-2.0, diffusers layout) is a partial copy of the base
MMDiT: its own input / context / time-text embedders, N joint blocks (6 shipped, no single blocks), a second input
embedder for the VAE-encoded control image added into the image stream, and one output projection per block. Block i's
projected image stream is residual i; the base transformer adds residual floor(i / interval) * control_scale to its image
stream after double block i, with interval = ceil(base double blocks / N).

Behaviour follows the reference's candle-gen-flux crate:
  - control.rs:1-640             branch layout, residual emission, the injection interval, accepted control kinds
  - ip_dit.rs:684-825            the base forward's seams: the post-block injector residual first, then the control residual
  - control_provider.rs:60-420   control image -> Lanczos resize -> [-1, 1] -> VAE posterior mean -> packed tokens; the
                                 dev schedule and guidance; default control scale 0.7 (an explicit 0 is honoured)

Here the branch's joint blocks are the base model's double blocks, so its checkpoint is converted once into the fused
FLUX layout (`convert_control_weights`) and the branch runs on the same model classes as the base (`OracleFluxDiT` on the
oracle backend, `FluxDiTGpu` with its tcgen05 GEMM / attention kernels on the device): the two input embedders become
one projection over the concatenated (latent, control) channels, and the per-block residuals are read at the model's
image-stream seam.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.runtime import CancelFlag
from ..models import nn_dual as nd
from ..models.dit_flux import FluxConfig

MODEL_ID = "flux1_dev_control"
DEFAULT_CONTROL_SCALE = 0.7
DEFAULT_STEPS, DEFAULT_GUIDANCE, SIZE_MULTIPLE = 25, 3.5, 16
CONTROL_KINDS = ("pose", "canny", "depth")
CONTROL_FILE = "diffusion_pytorch_model.safetensors"


def control_residual_interval(num_double_blocks: int, num_residuals: int) -> int:
    return -(-num_double_blocks // max(num_residuals, 1))


def accepts_control_kind(kind: str) -> bool:
    return kind in CONTROL_KINDS


def branch_layers(sd: dict[str, torch.Tensor]) -> int:
    n = 0
    while f"controlnet_blocks.{n}.weight" in sd:
        n += 1
    return n


def branch_config(base: FluxConfig, layers: int, guidance: bool = True) -> FluxConfig:
    """The branch shares the base's widths and rotary layout; its input is (latent ‖ control) channels."""
    return FluxConfig(in_channels=2 * base.in_channels, vec_in_dim=base.vec_in_dim, context_in_dim=base.context_in_dim,
                      hidden_size=base.hidden_size, mlp_ratio=base.mlp_ratio, num_heads=base.num_heads, depth=layers,
                      depth_single=0, axes_dim=base.axes_dim, theta=base.theta, guidance_embed=guidance)


def convert_control_weights(sd: dict[str, torch.Tensor], cfg: FluxConfig) -> tuple[dict[str, torch.Tensor], list[tuple]]:
    """diffusers `FluxControlNetModel` names -> (fused FLUX layout for a `cfg`-shaped model, per-block output projections).
    x_embedder and controlnet_x_embedder act on the same tokens and are summed, so they fuse into one projection of the
    concatenated channels; the model's final layer does not exist in the branch and is filled with zeros."""
    out: dict[str, torch.Tensor] = {}

    def need(k):
        if k not in sd:
            raise LoadError(f"{MODEL_ID}: control checkpoint lacks {k}")
        return sd[k]

    def take(dst, src):
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = need(f"{src}.{leaf}")

    def fuse(dst, srcs):
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = torch.cat([need(f"{s}.{leaf}") for s in srcs], dim=0)

    out["img_in.weight"] = torch.cat([need("x_embedder.weight"), need("controlnet_x_embedder.weight")], dim=1)
    out["img_in.bias"] = need("x_embedder.bias") + need("controlnet_x_embedder.bias")
    take("txt_in", "context_embedder")
    tte = "time_text_embed."
    take("time_in.in_layer", tte + "timestep_embedder.linear_1")
    take("time_in.out_layer", tte + "timestep_embedder.linear_2")
    take("vector_in.in_layer", tte + "text_embedder.linear_1")
    take("vector_in.out_layer", tte + "text_embedder.linear_2")
    if cfg.guidance_embed:
        take("guidance_in.in_layer", tte + "guidance_embedder.linear_1")
        take("guidance_in.out_layer", tte + "guidance_embedder.linear_2")
    for i in range(cfg.depth):
        s, d = f"transformer_blocks.{i}", f"double_blocks.{i}"
        take(f"{d}.img_mod.lin", f"{s}.norm1.linear")
        take(f"{d}.txt_mod.lin", f"{s}.norm1_context.linear")
        fuse(f"{d}.img_attn.qkv", [f"{s}.attn.to_q", f"{s}.attn.to_k", f"{s}.attn.to_v"])
        fuse(f"{d}.txt_attn.qkv", [f"{s}.attn.add_q_proj", f"{s}.attn.add_k_proj", f"{s}.attn.add_v_proj"])
        take(f"{d}.img_attn.proj", f"{s}.attn.to_out.0")
        take(f"{d}.txt_attn.proj", f"{s}.attn.to_add_out")
        out[f"{d}.img_attn.norm.query_norm.scale"] = need(f"{s}.attn.norm_q.weight")
        out[f"{d}.img_attn.norm.key_norm.scale"] = need(f"{s}.attn.norm_k.weight")
        out[f"{d}.txt_attn.norm.query_norm.scale"] = need(f"{s}.attn.norm_added_q.weight")
        out[f"{d}.txt_attn.norm.key_norm.scale"] = need(f"{s}.attn.norm_added_k.weight")
        take(f"{d}.img_mlp.0", f"{s}.ff.net.0.proj")
        take(f"{d}.img_mlp.2", f"{s}.ff.net.2")
        take(f"{d}.txt_mlp.0", f"{s}.ff_context.net.0.proj")
        take(f"{d}.txt_mlp.2", f"{s}.ff_context.net.2")
    H, ref = cfg.hidden_size, out["img_in.weight"]
    out["final_layer.adaLN_modulation.1.weight"] = ref.new_zeros(2 * H, H)
    out["final_layer.adaLN_modulation.1.bias"] = ref.new_zeros(2 * H)
    out["final_layer.linear.weight"] = ref.new_zeros(cfg.in_channels, H)
    out["final_layer.linear.bias"] = ref.new_zeros(cfg.in_channels)
    heads = [(need(f"controlnet_blocks.{i}.weight"), need(f"controlnet_blocks.{i}.bias")) for i in range(cfg.depth)]
    return out, heads


class _Capture:
    """Image-stream seam of the branch model: records each block's projected image stream, changes nothing."""

    def __init__(self, heads):
        self.heads, self.residuals = heads, []

    def after_double(self, i, img):
        w, b = self.heads[i]
        self.residuals.append(nd.linear(img, w, b))
        return None

    def after_single(self, i, img):
        return None


class _Residuals:
    """Image-stream seam of the base model: an optional inner injector's residual first, then the control residual."""

    def __init__(self, residuals, scale: float, interval: int, inner=None):
        self.residuals, self.scale, self.interval, self.inner = residuals, scale, interval, inner

    def after_double(self, i, img):
        r = self.inner.after_double(i, img) if self.inner is not None else None
        c = self.residuals[min(i // self.interval, len(self.residuals) - 1)] * self.scale
        return c if r is None else r.to(c.dtype) + c

    def after_single(self, i, img):
        return self.inner.after_single(i, img) if self.inner is not None else None


class FluxControlNet:
    """The control branch on the base model's classes. forward(...) -> one residual [B, S_img, hidden] per block."""

    def __init__(self, base_cfg: FluxConfig, sd: dict[str, torch.Tensor], device="cpu", guidance: bool = True):
        from ..models.dit_flux import FluxDiTGpu, OracleFluxDiT

        layers = branch_layers(sd)
        if layers == 0:
            raise LoadError(f"{MODEL_ID}: the control checkpoint has no controlnet_blocks")
        self.cfg = branch_config(base_cfg, layers, guidance)
        self.device = torch.device(device)
        weights, heads = convert_control_weights(sd, self.cfg)
        if self.device.type == "cuda":
            self.model = FluxDiTGpu(self.cfg, device=self.device).load_state_dict(weights)
            dt = torch.bfloat16
        else:
            self.model = OracleFluxDiT(self.cfg, weights, torch.float32, self.device)
            dt = torch.float32
        self.heads = [(w.to(self.device, dt).contiguous(), b.to(self.device, dt).contiguous()) for w, b in heads]

    @property
    def num_residuals(self) -> int:
        return len(self.heads)

    @torch.no_grad()
    def forward(self, img, control_cond, img_ids, txt, txt_ids, timesteps, y, guidance=None, rope=None) -> list[torch.Tensor]:
        cap = _Capture(self.heads)
        self.model.injector = cap
        try:
            x = torch.cat([img, control_cond.to(img.dtype)], dim=-1)
            if self.device.type == "cuda":
                self.model.forward(x, img_ids, txt, txt_ids, timesteps, y, guidance, rope=rope)
            else:
                self.model.forward(x, img_ids, txt, txt_ids, timesteps, y, guidance)
        finally:
            self.model.injector = None
        return cap.residuals


class ControlledDit:
    """Stands in for the base model during one render: every evaluation first runs the branch on the same inputs, then
    the base with the residual seam installed (and the caller's own injector, when there is one, ahead of it)."""

    def __init__(self, base, branch: FluxControlNet, control_cond: torch.Tensor, scale: float, inner=None):
        self.base, self.branch, self.control_cond, self.scale, self.inner = base, branch, control_cond, scale, inner
        self.interval = control_residual_interval(base.cfg.depth, branch.num_residuals)

    def __getattr__(self, name):
        return getattr(self.base, name)

    def _run(self, fn, img, img_ids, txt, txt_ids, timesteps, y, guidance=None, **kw):
        res = self.branch.forward(img, self.control_cond, img_ids, txt, txt_ids, timesteps, y, guidance, kw.get("rope"))
        self.base.injector = _Residuals(res, self.scale, self.interval, self.inner)
        try:
            return fn(img, img_ids, txt, txt_ids, timesteps, y, guidance, **kw)
        finally:
            self.base.injector = None

    def forward(self, *a, **kw):
        return self._run(self.base.forward, *a, **kw)

    def forward_graphed(self, *a, **kw):          # the residuals change every step: the eager path
        return self._run(self.base.forward, *a, **kw)


# ---- provider ---------------------------------------------------------------------------------------------------------------
@dataclass
class Flux1ControlPaths:
    flux_base: Path
    control: Path          # the branch checkpoint: a .safetensors file or a directory holding diffusion_pytorch_model.safetensors


@dataclass
class Flux1ControlRequest:
    prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int = DEFAULT_STEPS
    guidance: float = DEFAULT_GUIDANCE
    control_scale: float | None = None          # None -> DEFAULT_CONTROL_SCALE; an explicit 0.0 switches the control off
    control_kind: str = "pose"
    seed: int = 0
    cancel: CancelFlag = field(default_factory=CancelFlag)


class Flux1DevControl:
    def __init__(self, flux, branch: FluxControlNet, backend: str):
        self.flux, self.branch, self.backend = flux, branch, backend

    @staticmethod
    def load(paths: Flux1ControlPaths, backend: str = "b200") -> "Flux1DevControl":
        from ..contracts.gen_core.runtime import LoadSpec
        from ..io.safetensors_io import load_file
        from .catalog import provider_registry

        ctrl = Path(paths.control)
        if ctrl.is_dir():
            ctrl = ctrl / CONTROL_FILE
        if not ctrl.is_file():
            raise LoadError(f"{MODEL_ID}: control checkpoint {ctrl} not found")
        prefix = "" if backend == "b200" else "cpu_"
        flux = provider_registry(backend).load(prefix + "flux1_dev", LoadSpec.from_dir(paths.flux_base))
        sd = load_file(ctrl)
        guidance = any(k.startswith("time_text_embed.guidance_embedder.") for k in sd)
        branch = FluxControlNet(flux.pipe.dit_cfg, sd, "cuda" if backend == "b200" else "cpu", guidance)
        return Flux1DevControl(flux, branch, backend)

    @property
    def num_residuals(self) -> int:
        return self.branch.num_residuals

    @property
    def residual_interval(self) -> int:
        return control_residual_interval(self.flux.pipe.dit_cfg.depth, self.branch.num_residuals)

    def encode_control_latent(self, image: Image, width: int, height: int) -> torch.Tensor:
        """-> packed control tokens [1, (h/16)(w/16), 64]: the VAE posterior mean of the control image, shifted and scaled
        like any latent, in the DiT's 2 x 2 patch layout."""
        from ..io.safetensors_io import load_file
        from .flux import patchify
        from .reference import encode_reference_image

        if len(image.pixels) != image.width * image.height * 3:
            raise InferenceError(f"{MODEL_ID}: control pixel buffer {len(image.pixels)} != {image.width}x{image.height}x3")
        pipe = self.flux.pipe
        return patchify(encode_reference_image(pipe.vae_cfg, load_file(pipe.root / "ae.safetensors"), image, width, height,
                                               pipe.device, MODEL_ID))

    def generate(self, req: Flux1ControlRequest, control_image: Image, on_progress=lambda p: None, injector=None) -> Image:
        if req.cancel.is_cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        if not req.prompt.strip():
            raise InferenceError(f"{MODEL_ID}: prompt is required")
        if not accepts_control_kind(req.control_kind):
            raise InferenceError(f"{MODEL_ID} supports pose / canny / depth control, got {req.control_kind!r}")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{MODEL_ID}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.steps == 0:
            raise InferenceError(f"{MODEL_ID}: steps must be >= 1")
        scale = DEFAULT_CONTROL_SCALE if req.control_scale is None else float(req.control_scale)
        if not math.isfinite(scale):
            raise InferenceError(f"{MODEL_ID}: control_scale must be finite")
        gen, pipe = self.flux, self.flux.pipe
        greq = GenerationRequest(prompt=req.prompt, width=req.width, height=req.height, steps=req.steps, guidance=req.guidance,
                                 seed=req.seed, cancel=req.cancel)
        gen.validate(greq)

        def render(heavy, cond):
            control = self.encode_control_latent(control_image, req.width, req.height).to(heavy.device, heavy.dtype)
            base = heavy.dit
            heavy.dit = ControlledDit(base, self.branch, control, scale, injector)
            try:
                return pipe.render(heavy, cond, greq, on_progress)
            finally:
                heavy.dit = base

        return gen.residency.run(req.cancel, on_progress, lambda text: pipe.encode(text, req.prompt), render)[0]


# ---- synthetic checkpoint ---------------------------------------------------------------------------------------------------
def random_control_weights(base: FluxConfig, layers: int = 2, seed: int = 0, std: float = 0.05, zero_init: bool = False
                           ) -> dict[str, torch.Tensor]:
    """A branch checkpoint in the diffusers layout. zero_init reproduces the published initialisation (control embedder
    and output projections at zero: the branch then emits zero residuals)."""
    g = torch.Generator().manual_seed(seed)
    H, M = base.hidden_size, base.mlp_hidden
    w: dict[str, torch.Tensor] = {}

    def lin(name, o, i, zero=False):
        w[name + ".weight"] = torch.zeros(o, i) if zero else torch.randn(o, i, generator=g) * std
        w[name + ".bias"] = torch.zeros(o) if zero else torch.randn(o, generator=g) * std

    lin("x_embedder", H, base.in_channels)
    lin("controlnet_x_embedder", H, base.in_channels, zero_init)
    lin("context_embedder", H, base.context_in_dim)
    for n, d in (("timestep_embedder", 256), ("text_embedder", base.vec_in_dim), ("guidance_embedder", 256)):
        lin(f"time_text_embed.{n}.linear_1", H, d)
        lin(f"time_text_embed.{n}.linear_2", H, H)
    for i in range(layers):
        s = f"transformer_blocks.{i}"
        lin(f"{s}.norm1.linear", 6 * H, H)
        lin(f"{s}.norm1_context.linear", 6 * H, H)
        for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
            lin(f"{s}.attn.{n}", H, H)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            w[f"{s}.attn.{n}.weight"] = 1.0 + 0.1 * torch.randn(base.head_dim, generator=g)
        for ff in ("ff", "ff_context"):
            lin(f"{s}.{ff}.net.0.proj", M, H)
            lin(f"{s}.{ff}.net.2", H, M)
        lin(f"controlnet_blocks.{i}", H, H, zero_init)
    return w
