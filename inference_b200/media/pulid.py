"""PuLID-FLUX identity provider (parity: candle-gen-pulid/src/{pulid_flux,idformer,ca}.rs and eva_clip/*).

A reference face steers a FLUX.1-dev render: the face stack finds and embeds the face (ArcFace, 512 numbers), the aligned
crop is parsed and background-whitened, an EVA02-CLIP-L/14-336 tower reads it (class-token projection, 768 numbers, plus
the token states entering blocks 4, 8, 12, 16, 20), and the IDFormer (a perceiver resampler: 32 learned queries + 5
identity tokens attend the mapped tower states over ten layers, two per scale) fuses both into a 32 x 2048 identity
embedding. Twenty perceiver cross-attention modules then add `id_weight * attention(image tokens -> identity
embedding)` to the image stream of the DiT, after every second double block and every fourth single block.

Like the other identity providers this is a plain class driven directly by a caller (the registered `flux1_*`
generators stay text-to-image); it holds a FLUX generator of this package and installs its hooks through the DiT's
`injector` seam for the duration of one request, so both backends (and the tcgen05 kernels of the DiT) are reused.
The small identity networks run in fp32 through the framework's tensor ops."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from ..contracts.errors import Canceled, InferenceError, LoadError
from ..contracts.gen_core.generator import GenerationRequest
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.runtime import CancelFlag

SIZE_MULTIPLE, DEFAULT_ID_WEIGHT, DEFAULT_GUIDANCE, DEFAULT_STEPS = 16, 1.0, 4.0, 25
EVA_MEAN, EVA_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)
LN_EPS, EVA_EPS, LEAKY = 1e-5, 1e-6, 0.01


# ---- EVA02-CLIP vision tower ----------------------------------------------------------------------------------------------
@dataclass
class EvaConfig:
    image_size: int = 336
    patch: int = 14
    embed_dim: int = 1024
    depth: int = 24
    num_heads: int = 16
    proj_dim: int = 768
    pt_seq_len: int = 16
    rope_theta: float = 10000.0
    hidden_capture: tuple = (4, 8, 12, 16, 20)
    mlp_dim: int = 2730

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def grid(self) -> int:
        return self.image_size // self.patch


def eva_rope_tables(head_dim: int, grid: int, pt_seq_len: int, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [grid * grid, head_dim]: first half of the head follows the row, second half the column; positions are
    rescaled onto the pre-training grid (i / grid * pt_seq_len); every frequency fills an adjacent pair."""
    half = head_dim // 2
    freqs = 1.0 / theta ** (torch.arange(0, half, 2, dtype=torch.float64) / half)
    t = torch.arange(grid, dtype=torch.float64) / grid * pt_seq_len
    axis = (t[:, None] * freqs[None]).repeat_interleave(2, dim=1)               # [grid, half]
    ang = torch.cat([axis[:, None, :].expand(grid, grid, half), axis[None, :, :].expand(grid, grid, half)], -1)
    ang = ang.reshape(grid * grid, head_dim)
    return ang.cos().float(), ang.sin().float()


def rotate_pairs(x: torch.Tensor) -> torch.Tensor:
    """(x0, x1, x2, x3, ...) -> (-x1, x0, -x3, x2, ...)."""
    xr = x.reshape(*x.shape[:-1], -1, 2)
    return torch.stack([-xr[..., 1], xr[..., 0]], -1).reshape(x.shape)


class EvaVisionTower:
    def __init__(self, weights: dict[str, torch.Tensor], cfg: EvaConfig | None = None, device="cpu", prefix: str = ""):
        self.cfg, self.device = cfg or EvaConfig(), torch.device(device)
        self.w = {k[len(prefix):]: v.float().to(self.device) for k, v in weights.items() if k.startswith(prefix)}
        pw = self.w["patch_embed.proj.weight"]
        if pw.shape[-1] == 3 and pw.shape[1] != 3:                   # stored [out, kh, kw, in]
            self.w["patch_embed.proj.weight"] = pw.permute(0, 3, 1, 2).contiguous()
        c = self.cfg
        self.cos, self.sin = (t.to(self.device) for t in eva_rope_tables(c.head_dim, c.grid, c.pt_seq_len, c.rope_theta))

    def _ln(self, x, p):
        return F.layer_norm(x, (x.shape[-1],), self.w[p + ".weight"], self.w[p + ".bias"], EVA_EPS)

    def _lin(self, x, p, bias=None):
        return F.linear(x, self.w[p + ".weight"], self.w.get(p + ".bias") if bias is None else bias)

    def _rope(self, x):                                       # [B, H, N, hd]: the class token keeps its place
        pat = x[:, :, 1:]
        return torch.cat([x[:, :, :1], pat * self.cos + rotate_pairs(pat) * self.sin], 2)

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> tuple[torch.Tensor, list[torch.Tensor]]:
        """[B, 3, S, S] normalised -> (class projection [B, proj_dim], the states entering the captured blocks)."""
        c, w = self.cfg, self.w
        x = F.conv2d(pixels.to(self.device), w["patch_embed.proj.weight"], w["patch_embed.proj.bias"], stride=c.patch)
        B = x.shape[0]
        x = torch.cat([w["cls_token"].expand(B, 1, -1), x.flatten(2).transpose(1, 2)], 1) + w["pos_embed"]
        H, hd = c.num_heads, c.head_dim
        hidden = []
        for i in range(c.depth):
            if i in c.hidden_capture:
                hidden.append(x)
            p = f"blocks.{i}"
            h = self._ln(x, p + ".norm1")
            heads = lambda t: t.view(B, -1, H, hd).transpose(1, 2)                       # noqa: E731
            q = self._rope(heads(self._lin(h, p + ".attn.q_proj", w[p + ".attn.q_bias"])))
            k = self._rope(heads(F.linear(h, w[p + ".attn.k_proj.weight"])))
            v = heads(self._lin(h, p + ".attn.v_proj", w[p + ".attn.v_bias"]))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, -1, H * hd)
            x = x + self._lin(self._ln(a, p + ".attn.inner_attn_ln"), p + ".attn.proj")
            h = self._ln(x, p + ".norm2")
            g = F.silu(self._lin(h, p + ".mlp.w1")) * self._lin(h, p + ".mlp.w2")
            x = x + self._lin(self._ln(g, p + ".mlp.ffn_ln"), p + ".mlp.w3")
        cls = self._ln(x, "norm")[:, 0]
        return self._lin(cls, "head"), hidden


def _cubic(x: np.ndarray, a: float = -0.5) -> np.ndarray:
    x = np.abs(x)
    return np.where(x < 1.0, ((a + 2.0) * x - (a + 3.0)) * x * x + 1.0, np.where(x < 2.0, (((x - 5.0) * x + 8.0) * x - 4.0) * a, 0.0))


def _resize_matrix(n_in: int, n_out: int) -> np.ndarray:
    """Antialiased bicubic (Keys a = -0.5) resampling weights [n_out, n_in], the Pillow convention."""
    scale = n_in / n_out
    fs = max(scale, 1.0)
    support = 2.0 * fs
    m = np.zeros((n_out, n_in), dtype=np.float64)
    for i in range(n_out):
        centre = (i + 0.5) * scale
        lo = max(int(math.floor(centre - support + 0.5)), 0)
        hi = min(int(math.floor(centre + support + 0.5)), n_in)
        wts = _cubic((np.arange(lo, hi) - centre + 0.5) / fs)
        tot = wts.sum()
        m[i, lo:hi] = wts / tot if tot != 0 else wts
    return m


def eva_transform(rgb01: torch.Tensor, size: int) -> torch.Tensor:
    """[1, 3, H, W] in [0, 1] -> [1, 3, size, size]: antialiased bicubic resize (rows then columns), CLIP mean / std."""
    if rgb01.shape[0] != 1:
        raise InferenceError(f"eva_transform handles a single image, got batch {rgb01.shape[0]}")
    x = rgb01[0].double().cpu()
    mh = torch.from_numpy(_resize_matrix(x.shape[1], size))
    mw = torch.from_numpy(_resize_matrix(x.shape[2], size))
    y = (x @ mw.t()).float().double()                         # the horizontal pass is stored in fp32 between the passes
    y = (mh @ y).float()
    mean, std = torch.tensor(EVA_MEAN).view(3, 1, 1), torch.tensor(EVA_STD).view(3, 1, 1)
    return ((y - mean) / std)[None]


# ---- IDFormer -----------------------------------------------------------------------------------------------------------
@dataclass
class IdFormerConfig:
    dim: int = 1024
    depth: int = 10
    heads: int = 16
    dim_head: int = 64
    num_id_token: int = 5
    num_queries: int = 32
    output_dim: int = 2048
    id_dim: int = 1280            # ArcFace 512 + tower projection 768
    vit_dim: int = 1024


class _Net:
    def __init__(self, weights, device, prefix=""):
        self.device = torch.device(device)
        self.w = {k[len(prefix):]: v.float().to(self.device) for k, v in weights.items() if k.startswith(prefix)}

    def lin(self, x, p):
        return F.linear(x, self.w[p + ".weight"], self.w.get(p + ".bias"))

    def ln(self, x, p):
        return F.layer_norm(x, (x.shape[-1],), self.w[p + ".weight"], self.w[p + ".bias"], LN_EPS)


def perceiver_attention(net: _Net, p: str, ctx: torch.Tensor, lat: torch.Tensor, heads: int, dim_head: int, self_kv: bool):
    """Queries from norm2(lat); keys / values from norm1(ctx) (followed by the normalised latents when `self_kv`)."""
    x, l = net.ln(ctx, p + ".norm1"), net.ln(lat, p + ".norm2")
    B, n = l.shape[:2]
    q = net.lin(l, p + ".to_q")
    kv = net.lin(torch.cat([x, l], 1) if self_kv else x, p + ".to_kv")
    k, v = kv.chunk(2, -1)
    hs = lambda t: t.view(B, -1, heads, dim_head).transpose(1, 2)                        # noqa: E731
    o = F.scaled_dot_product_attention(hs(q), hs(k), hs(v)).transpose(1, 2).reshape(B, n, heads * dim_head)
    return net.lin(o, p + ".to_out")


class IdFormer(_Net):
    def __init__(self, weights, cfg: IdFormerConfig | None = None, device="cpu", prefix: str = "pulid_encoder."):
        super().__init__(weights, device, prefix)
        self.cfg = cfg or IdFormerConfig()

    def _mapping(self, x, p):
        h = F.leaky_relu(self.ln(self.lin(x, p + ".0"), p + ".1"), LEAKY)
        h = F.leaky_relu(self.ln(self.lin(h, p + ".3"), p + ".4"), LEAKY)
        return self.lin(h, p + ".6")

    @torch.no_grad()
    def forward(self, id_cond: torch.Tensor, vit_hidden: list[torch.Tensor]) -> torch.Tensor:
        """id_cond [B, id_dim], five tower states [B, N, vit_dim] -> the identity embedding [B, num_queries, output_dim]."""
        c = self.cfg
        if len(vit_hidden) != 5:
            raise InferenceError(f"IDFormer expects 5 EVA hidden states, got {len(vit_hidden)}")
        B = id_cond.shape[0]
        x = self._mapping(id_cond.to(self.device), "id_embedding_mapping").view(B, c.num_id_token, c.dim)
        lat = torch.cat([self.w["latents"].expand(B, -1, -1), x], 1)
        per = c.depth // 5
        for i, h in enumerate(vit_hidden):
            ctx = torch.cat([x, self._mapping(h.to(self.device), f"mapping_{i}")], 1)
            for layer in range(i * per, (i + 1) * per):
                lat = lat + perceiver_attention(self, f"layers.{layer}.0", ctx, lat, c.heads, c.dim_head, True)
                f = f"layers.{layer}.1"
                lat = lat + F.linear(F.gelu(F.linear(self.ln(lat, f + ".0"), self.w[f + ".1.weight"])), self.w[f + ".3.weight"])
        return lat[:, :c.num_queries] @ self.w["proj_out"]


class PulidCa(_Net):
    """The DiT image-stream hooks: module k serves double block 2k; after the double blocks, single block 4k."""

    def __init__(self, weights, id_embedding: torch.Tensor, id_weight: float, num_double: int, num_single: int, device="cpu",
                 prefix: str = "pulid_ca.", heads: int = 16, dim_head: int = 128):
        super().__init__(weights, device, prefix)
        if "swb_ca_config" in weights:                        # synthetic checkpoints carry their head geometry
            heads, dim_head = (int(v) for v in weights["swb_ca_config"].tolist())
        self.id, self.id_weight = id_embedding.float().to(self.device), float(id_weight)
        self.double_interval, self.single_interval = 2, 4
        self.n_double = -(-num_double // self.double_interval)
        self.num_ca = self.n_double + -(-num_single // self.single_interval)
        self.heads, self.dim_head = heads, dim_head

    def _ca(self, k: int, img: torch.Tensor) -> torch.Tensor:
        x = img.float().to(self.device)
        return perceiver_attention(self, str(k), self.id.expand(x.shape[0], -1, -1), x, self.heads, self.dim_head, False) * self.id_weight

    def after_double(self, i: int, img: torch.Tensor):
        if self.id_weight == 0.0 or i % self.double_interval:
            return None
        return self._ca(i // self.double_interval, img)

    def after_single(self, i: int, img: torch.Tensor):
        if self.id_weight == 0.0 or i % self.single_interval:
            return None
        return self._ca(self.n_double + i // self.single_interval, img)


# ---- provider -----------------------------------------------------------------------------------------------------------
@dataclass
class PulidFluxPaths:
    flux_base: Path
    pulid_weights: Path
    eva_weights: Path
    face_dir: Path


@dataclass
class PulidFluxRequest:
    prompt: str = ""
    width: int = 1024
    height: int = 1024
    steps: int = DEFAULT_STEPS
    guidance: float = DEFAULT_GUIDANCE
    id_weight: float = DEFAULT_ID_WEIGHT
    sampler: str | None = None
    scheduler: str | None = None
    seed: int = 0
    cancel: CancelFlag = field(default_factory=CancelFlag)


def reject_below_floor(req: PulidFluxRequest) -> None:
    if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
        raise InferenceError(f"pulid_flux: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
    if req.steps == 0:
        raise InferenceError("pulid_flux: steps must be >= 1 (an explicit 0 renders undenoised noise)")


def l2_normalize_rows(x: torch.Tensor) -> torch.Tensor:
    return x / x.pow(2).sum(1, keepdim=True).sqrt().clamp(min=1e-12)


class PulidFlux:
    def __init__(self, flux, eva: EvaVisionTower, idformer: IdFormer, pulid_weights: dict, face, parser, backend: str):
        self.flux, self.eva, self.idformer, self.pulid, self.face, self.parser, self.backend = \
            flux, eva, idformer, pulid_weights, face, parser, backend

    @staticmethod
    def load(paths: PulidFluxPaths, backend: str = "b200") -> "PulidFlux":
        from ..contracts.gen_core.runtime import LoadSpec
        from ..io.safetensors_io import load_file
        from . import face as face_mod
        from .catalog import provider_registry

        for what, f in (("EVA weights", paths.eva_weights), ("PuLID weights", paths.pulid_weights)):
            if not Path(f).is_file():
                raise LoadError(f"pulid_flux: load {what} {f}: file not found")
        prefix = "" if backend == "b200" else "cpu_"
        dev = "cuda" if backend == "b200" else "cpu"
        flux = provider_registry(backend).load(prefix + "flux1_dev", LoadSpec.from_dir(paths.flux_base))
        eva_w, pulid_w = load_file(paths.eva_weights), load_file(paths.pulid_weights)
        cfg = EvaConfig()
        if "swb_eva_config" in eva_w:                         # synthetic checkpoints carry their dimensions
            v = [int(t) for t in eva_w.pop("swb_eva_config").tolist()]
            cfg = EvaConfig(image_size=v[0], patch=v[1], embed_dim=v[2], depth=v[3], num_heads=v[4], proj_dim=v[5], pt_seq_len=v[6],
                            hidden_capture=tuple(v[7:12]), mlp_dim=v[12])
        icfg = IdFormerConfig()
        if "swb_idformer_config" in pulid_w:
            v = [int(t) for t in pulid_w.pop("swb_idformer_config").tolist()]
            icfg = IdFormerConfig(*v)
        pulid_w = {k: v for k, v in pulid_w.items()}
        bis = Path(paths.face_dir) / face_mod.BISENET_FILE
        if not bis.is_file():
            raise LoadError(f"pulid_flux: {bis} not found (the face-parsing checkpoint)")
        return PulidFlux(flux, EvaVisionTower(eva_w, cfg, dev), IdFormer(pulid_w, icfg, dev), pulid_w,
                         face_mod.load(paths.face_dir, backend), face_mod.BiSeNet(load_file(bis), dev), backend)

    def compute_id_embedding(self, reference: Image) -> torch.Tensor:
        from . import face as face_mod

        faces = self.face.analyze(reference)
        if not faces:
            raise InferenceError("pulid_flux: no face detected in the reference image")
        f = faces[0]
        arc = torch.tensor([f.embedding], dtype=torch.float32)
        ffi = face_mod.face_features_for(self.face, self.parser, reference, f)
        proj, hidden = self.eva.forward(eva_transform(ffi, self.eva.cfg.image_size))
        id_cond = torch.cat([arc.to(proj.device), l2_normalize_rows(proj)], 1)
        return self.idformer.forward(id_cond, hidden)

    def generate(self, req: PulidFluxRequest, reference: Image, on_progress=lambda p: None) -> Image:
        if req.cancel.is_cancelled():
            raise Canceled("pulid_flux: cancelled")
        reject_below_floor(req)
        id_embedding = self.compute_id_embedding(reference)
        gen, pipe = self.flux, self.flux.pipe
        greq = GenerationRequest(prompt=req.prompt, width=req.width, height=req.height, steps=req.steps, guidance=req.guidance,
                                 sampler=req.sampler, scheduler=req.scheduler, seed=req.seed, cancel=req.cancel)
        gen.validate(greq)

        def render(heavy, cond):
            cfg = pipe.dit_cfg
            heavy.dit.injector = PulidCa(self.pulid, id_embedding, req.id_weight, cfg.depth, cfg.depth_single, pipe.device)
            try:
                return pipe.render(heavy, cond, greq, on_progress)
            finally:
                heavy.dit.injector = None

        return gen.residency.run(req.cancel, on_progress, lambda text: pipe.encode(text, req.prompt), render)[0]


# ---- synthetic checkpoints ------------------------------------------------------------------------------------------------
def random_eva_weights(cfg: EvaConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                    # noqa: E731
    w: dict[str, torch.Tensor] = {}
    D = cfg.embed_dim

    def lin(p, o, i, bias=True):
        w[p + ".weight"] = rn(o, i) / math.sqrt(i)
        if bias:
            w[p + ".bias"] = rn(o) * 0.02

    def ln(p, d):
        w[p + ".weight"], w[p + ".bias"] = 1 + rn(d) * 0.05, rn(d) * 0.02

    w["patch_embed.proj.weight"] = rn(D, cfg.patch, cfg.patch, 3) / math.sqrt(3 * cfg.patch ** 2)
    w["patch_embed.proj.bias"] = rn(D) * 0.02
    w["cls_token"], w["pos_embed"] = rn(1, 1, D) * 0.1, rn(1, cfg.grid ** 2 + 1, D) * 0.1
    for i in range(cfg.depth):
        p = f"blocks.{i}"
        ln(p + ".norm1", D)
        ln(p + ".norm2", D)
        for n in ("q_proj", "k_proj", "v_proj"):
            lin(f"{p}.attn.{n}", D, D, bias=False)
        w[p + ".attn.q_bias"], w[p + ".attn.v_bias"] = rn(D) * 0.02, rn(D) * 0.02
        ln(p + ".attn.inner_attn_ln", D)
        lin(p + ".attn.proj", D, D)
        lin(p + ".mlp.w1", cfg.mlp_dim, D)
        lin(p + ".mlp.w2", cfg.mlp_dim, D)
        ln(p + ".mlp.ffn_ln", cfg.mlp_dim)
        lin(p + ".mlp.w3", D, cfg.mlp_dim)
    ln("norm", D)
    lin("head", cfg.proj_dim, D)
    return w


def random_pulid_weights(cfg: IdFormerConfig, hidden: int, num_ca: int, seed: int = 0, ca_heads: int = 2, ca_dim_head: int = 8
                         ) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)                    # noqa: E731
    w: dict[str, torch.Tensor] = {}

    def lin(p, o, i, bias=True):
        w[p + ".weight"] = rn(o, i) / math.sqrt(i)
        if bias:
            w[p + ".bias"] = rn(o) * 0.02

    def ln(p, d):
        w[p + ".weight"], w[p + ".bias"] = 1 + rn(d) * 0.05, rn(d) * 0.02

    def mapping(p, i, o):
        lin(p + ".0", cfg.dim, i)
        ln(p + ".1", cfg.dim)
        lin(p + ".3", cfg.dim, cfg.dim)
        ln(p + ".4", cfg.dim)
        lin(p + ".6", o, cfg.dim)

    e = "pulid_encoder."
    w[e + "latents"], w[e + "proj_out"] = rn(1, cfg.num_queries, cfg.dim) * 0.1, rn(cfg.dim, cfg.output_dim) / math.sqrt(cfg.dim)
    mapping(e + "id_embedding_mapping", cfg.id_dim, cfg.dim * cfg.num_id_token)
    for i in range(5):
        mapping(e + f"mapping_{i}", cfg.vit_dim, cfg.dim)
    inner = cfg.heads * cfg.dim_head
    for i in range(cfg.depth):
        p = e + f"layers.{i}.0"
        ln(p + ".norm1", cfg.dim)
        ln(p + ".norm2", cfg.dim)
        lin(p + ".to_q", inner, cfg.dim, bias=False)
        lin(p + ".to_kv", 2 * inner, cfg.dim, bias=False)
        lin(p + ".to_out", cfg.dim, inner, bias=False)
        f = e + f"layers.{i}.1"
        ln(f + ".0", cfg.dim)
        lin(f + ".1", 4 * cfg.dim, cfg.dim, bias=False)
        lin(f + ".3", cfg.dim, 4 * cfg.dim, bias=False)
    inner = ca_heads * ca_dim_head
    for k in range(num_ca):
        p = f"pulid_ca.{k}"
        ln(p + ".norm1", cfg.output_dim)
        ln(p + ".norm2", hidden)
        lin(p + ".to_q", inner, hidden, bias=False)
        lin(p + ".to_kv", 2 * inner, cfg.output_dim, bias=False)
        lin(p + ".to_out", hidden, inner, bias=False)
    return w
