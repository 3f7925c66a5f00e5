"""FLUX.1 with the XLabs IP-Adapter (image-prompt conditioning): a bespoke provider driven by name.

A reference image goes through CLIP ViT-L/14 (class token -> post layer norm -> visual projection, 768 wide, not
normalised), a projection turns that vector into 4 tokens of width 4096, and every double block owns a key and a value
projection of those tokens. Inside block i the image stream's query (after its q norm, before rotation) attends to the
4 image-prompt tokens; the result, times `ip_adapter_scale`, is added to the image stream at the end of the block.
Scale 0 is the base model, bit for bit.

Behaviour follows the reference's candle-gen-flux crate:
  - ip_adapter.rs:10-230        the projection model (LayerNorm eps 1e-5), 19 (k, v) pairs, the per-block residual, keys
                                and values computed once per generation
  - ip_dit.rs:395-470           where the query is taken and where the residual lands in the double block
  - ip_image_encoder.rs:10-60   the CLIP image embedding
  - ip_provider.rs:40-420       paths, request defaults (scale 0.7), variant detection, request checks

The seam is `on_img_query` / `after_double` of the base model classes (`models/dit_flux.py`), so the adapter runs on the
oracle backend and on the sm_100a model alike and composes with the other image-stream injectors.
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

MODEL_ID = "flux1_ip_adapter"
NUM_TOKENS, PROJ_LN_EPS = 4, 1e-5
DEFAULT_IP_SCALE, SIZE_MULTIPLE = 0.7, 16


class FluxIpAdapter:
    def __init__(self, weights: dict[str, torch.Tensor], device="cpu"):
        self.device = torch.device(device)
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        for k in ("ip_adapter_proj_model.proj.weight", "ip_adapter_proj_model.proj.bias", "ip_adapter_proj_model.norm.weight",
                  "ip_adapter_proj_model.norm.bias"):
            if k not in weights:
                raise LoadError(f"{MODEL_ID}: adapter checkpoint lacks {k}")
        self.w = nd.WeightBag(weights, self.dtype, self.device)
        self.blocks = 0
        while f"double_blocks.{self.blocks}.processor.ip_adapter_double_stream_k_proj.weight" in self.w:
            self.blocks += 1
        if self.blocks == 0:
            raise LoadError(f"{MODEL_ID}: adapter checkpoint has no double-block projections")
        self.cross_dim = self.w["ip_adapter_proj_model.norm.weight"].shape[0]
        if self.w["ip_adapter_proj_model.proj.weight"].shape[0] % self.cross_dim:
            raise LoadError(f"{MODEL_ID}: projection rows are not a whole number of {self.cross_dim}-wide tokens")
        self.num_tokens = self.w["ip_adapter_proj_model.proj.weight"].shape[0] // self.cross_dim

    def tokens(self, image_embeds: torch.Tensor) -> torch.Tensor:
        """[B, embed] -> [B, num_tokens, cross_dim]."""
        w = self.w
        x = w.lin(image_embeds.to(self.device, self.dtype), "ip_adapter_proj_model.proj")
        x = x.view(image_embeds.shape[0], self.num_tokens, self.cross_dim)
        return nd.layer_norm(x, w["ip_adapter_proj_model.norm.weight"], w["ip_adapter_proj_model.norm.bias"], PROJ_LN_EPS)

    def block_kv(self, i: int, tokens: torch.Tensor, heads: int, head_dim: int) -> tuple[torch.Tensor, torch.Tensor]:
        p = f"double_blocks.{i}.processor.ip_adapter_double_stream_"
        B, T = tokens.shape[:2]
        return (self.w.lin(tokens, p + "k_proj").view(B, T, heads, head_dim), self.w.lin(tokens, p + "v_proj").view(B, T, heads, head_dim))


class FluxIpInjector:
    """Per generation: the image-prompt tokens and, per block, their keys and values (computed at first use and kept for
    the remaining steps)."""

    def __init__(self, adapter: FluxIpAdapter, tokens: torch.Tensor, scale: float, inner=None):
        self.adapter, self.tokens, self.scale, self.inner = adapter, tokens, float(scale), inner
        self.kv: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        self.q: dict[int, torch.Tensor] = {}

    def on_img_query(self, i: int, q: torch.Tensor) -> None:
        if self.scale != 0.0 and i < self.adapter.blocks:
            self.q[i] = q

    def residual(self, i: int) -> torch.Tensor | None:
        q = self.q.pop(i, None)
        if q is None:
            return None
        if i not in self.kv:
            self.kv[i] = self.adapter.block_kv(i, self.tokens, q.shape[2], q.shape[3])
        k, v = self.kv[i]
        return nd.attention(q.contiguous(), k.to(q.dtype), v.to(q.dtype)) * self.scale

    def after_double(self, i: int, img: torch.Tensor):
        r = self.inner.after_double(i, img) if self.inner is not None else None
        c = self.residual(i)
        if c is None:
            return r
        return c if r is None else r.to(c.dtype) + c

    def after_single(self, i: int, img: torch.Tensor):
        return self.inner.after_single(i, img) if self.inner is not None else None


# ---- provider ---------------------------------------------------------------------------------------------------------------
@dataclass
class IpAdapterFluxPaths:
    flux_base: Path
    ip_adapter: Path          # ip_adapter.safetensors
    image_encoder: Path       # a CLIP ViT-L/14 snapshot directory (config.json + weights)


@dataclass
class IpAdapterFluxRequest:
    prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int | None = None           # None: the variant's default (dev 25-class schedules, schnell 4)
    guidance: float = 3.5              # embedded by the dev model, inert on schnell
    ip_adapter_scale: float = DEFAULT_IP_SCALE
    seed: int = 0
    cancel: CancelFlag = field(default_factory=CancelFlag)


def detect_variant(root: Path) -> str:
    root = Path(root)
    for name, mid in (("flux1-dev.safetensors", "flux1_dev"), ("flux1-schnell.safetensors", "flux1_schnell")):
        if (root / name).is_file():
            return mid
    raise LoadError(f"{MODEL_ID}: {root} holds neither flux1-dev.safetensors nor flux1-schnell.safetensors")


class IpAdapterFlux:
    def __init__(self, flux, adapter: FluxIpAdapter, clip, backend: str):
        self.flux, self.adapter, self.clip, self.backend = flux, adapter, clip, backend

    @staticmethod
    def load(paths: IpAdapterFluxPaths, backend: str = "b200") -> "IpAdapterFlux":
        from ..contracts.gen_core.runtime import LoadSpec
        from ..io.safetensors_io import load_file
        from .catalog import provider_registry

        if not Path(paths.ip_adapter).is_file():
            raise LoadError(f"{MODEL_ID}: load adapter {paths.ip_adapter}: file not found")
        prefix = "" if backend == "b200" else "cpu_"
        reg = provider_registry(backend)
        flux = reg.load(prefix + detect_variant(paths.flux_base), LoadSpec.from_dir(paths.flux_base))
        adapter = FluxIpAdapter(load_file(paths.ip_adapter), "cuda" if backend == "b200" else "cpu")
        if adapter.blocks != flux.pipe.dit_cfg.depth:
            raise LoadError(f"{MODEL_ID}: adapter has {adapter.blocks} double-block pairs but the DiT has "
                            f"{flux.pipe.dit_cfg.depth} double blocks")
        enc = Path(paths.image_encoder)
        clip = reg.load_kind("image_embedder", "clip_vit_l14", LoadSpec.from_dir(enc if enc.is_dir() else enc.parent))
        return IpAdapterFlux(flux, adapter, clip, backend)

    def image_embeds(self, reference: Image) -> torch.Tensor:
        """The reference's CLIP image embedding [1, projection dim] (class token, post norm, projection; not normalised)."""
        from .vision_providers import CLIP_MEAN, CLIP_STD, image_tensor, preprocess

        tower = self.clip.tower
        return tower.image_embeds(preprocess(image_tensor(reference), tower.cfg.image_size, CLIP_MEAN, CLIP_STD)).float()

    def generate(self, req: IpAdapterFluxRequest, reference: Image, on_progress=lambda p: None, injector=None) -> Image:
        if req.cancel.is_cancelled():
            raise Canceled(f"{MODEL_ID}: cancelled")
        if not req.prompt.strip():
            raise InferenceError(f"{MODEL_ID}: prompt is required")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{MODEL_ID}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.steps == 0:
            raise InferenceError(f"{MODEL_ID}: steps must be >= 1")
        if not math.isfinite(req.ip_adapter_scale):
            raise InferenceError(f"{MODEL_ID}: ip_adapter_scale must be finite")
        gen, pipe = self.flux, self.flux.pipe
        greq = GenerationRequest(prompt=req.prompt, width=req.width, height=req.height, steps=req.steps, seed=req.seed,
                                 guidance=req.guidance if pipe.variant.supports_guidance else None, cancel=req.cancel)
        gen.validate(greq)
        tokens = self.adapter.tokens(self.image_embeds(reference))

        def render(heavy, cond):
            heavy.dit.injector = FluxIpInjector(self.adapter, tokens, req.ip_adapter_scale, injector)
            try:
                return pipe.render(heavy, cond, greq, on_progress)
            finally:
                heavy.dit.injector = None

        return gen.residency.run(req.cancel, on_progress, lambda text: pipe.encode(text, req.prompt), render)[0]


# ---- synthetic checkpoint ---------------------------------------------------------------------------------------------------
def random_ip_adapter_weights(blocks: int, hidden: int, embed_dim: int, cross_dim: int = 32, num_tokens: int = NUM_TOKENS,
                              seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    w = {"ip_adapter_proj_model.proj.weight": rn(num_tokens * cross_dim, embed_dim) / math.sqrt(embed_dim),
         "ip_adapter_proj_model.proj.bias": rn(num_tokens * cross_dim) * 0.02,
         "ip_adapter_proj_model.norm.weight": 1 + rn(cross_dim) * 0.05, "ip_adapter_proj_model.norm.bias": rn(cross_dim) * 0.02}
    for i in range(blocks):
        for n in ("k_proj", "v_proj"):
            p = f"double_blocks.{i}.processor.ip_adapter_double_stream_{n}"
            w[p + ".weight"], w[p + ".bias"] = rn(hidden, cross_dim) / math.sqrt(cross_dim), rn(hidden) * 0.02
    return w
