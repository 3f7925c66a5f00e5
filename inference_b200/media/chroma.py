"""Chroma text-to-image providers `chroma1_hd`, `chroma1_base`, `chroma1_flash` (and `cpu_*` on the fp32 oracle)
(parity: candle-gen-chroma/src/lib.rs, pipeline.rs, beta.rs, text.rs).

generate(): T5 encode of the prompt (un-padded, as many tokens as the prompt has) and, when true-CFG guidance > 1,
of the negative prompt -> per image: seeded CPU noise -> 2x2 patchify -> flow-matching Euler over the variant's sigma
schedule (hd: linspace 1 -> 1/N time-shifted by 3; base: Beta(0.6, 0.6) quantile spacing; flash: plain linspace),
each step one DiT forward (two with true CFG: neg + g * (pos - neg)) -> unpatchify -> FLUX VAE -> RGB8.

Snapshot layout (diffusers): `transformer/` (Chroma DiT + config.json), `text_encoder/` (T5) + `tokenizer/`
(`spiece.model`), `vae/` (AutoencoderKL in diffusers key names, converted to the decoder's native names at load).
`swb_config.json` in the root overrides dimensions for synthetic snapshots, as for the FLUX providers."""
from __future__ import annotations

import enum
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch

from ..contracts.errors import Canceled, InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import (Capabilities, GenerationOutput, GenerationRequest, Generator, Modality,
                                            ModelDescriptor)
from ..contracts.gen_core.media import Image
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import LoadSpec, OffloadPolicy, ProgressDecoding, ProgressStep
from ..contracts.gen_core.sampling import SCHEDULERS, SOLVERS
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_chroma import ChromaConfig, OracleChromaDiT
from ..models.dit_flux import make_ids, rope_table
from ..models.vae import OracleVaeDecoder, VaeConfig
from .flux import SIZE_MULTIPLE, patchify, unpatchify
from .residency import Residency
from .seed import default_seed, for_each_image_seed, seeded_noise_nchw


class ChromaVariant(enum.Enum):
    HD = "chroma1_hd"
    BASE = "chroma1_base"
    FLASH = "chroma1_flash"

    @property
    def default_steps(self) -> int:
        return 8 if self is ChromaVariant.FLASH else 28

    @property
    def default_true_cfg(self) -> float:
        return 1.0 if self is ChromaVariant.FLASH else 4.0

    @property
    def sigma_shift(self) -> float:
        return 3.0 if self is ChromaVariant.HD else 1.0

    @property
    def use_beta_sigmas(self) -> bool:
        return self is ChromaVariant.BASE


# ---- sigma schedules ---------------------------------------------------------------------------------------------------------
def beta_ppf(p: float, a: float = 0.6) -> float:
    """Quantile of Beta(a, a)."""
    from ..contracts.gen_core.sampling.schedulers import beta_ppf as ppf

    return ppf(p, a, a)


def chroma_sigmas(variant: ChromaVariant, steps: int) -> list[float]:
    """steps + 1 values from 1 down to 0."""
    n = max(1, steps)
    smin = 1.0 / n
    lin = [0.0 if n == 1 else i / (n - 1) for i in range(n)]
    if variant.use_beta_sigmas:
        out = [smin + beta_ppf(1.0 - t) * (1.0 - smin) for t in lin]
    else:
        sh = variant.sigma_shift
        raw = [1.0 + (smin - 1.0) * t for t in lin]
        out = [sh * s / (1.0 + (sh - 1.0) * s) for s in raw]
    return out + [0.0]


# ---- checkpoint helpers ------------------------------------------------------------------------------------------------------
def convert_diffusers_vae_decoder(sd: dict[str, torch.Tensor], levels: int = 4) -> dict[str, torch.Tensor]:
    """AutoencoderKL decoder keys in diffusers naming -> the decoder's native (latent-diffusion) naming; the mid-block
    attention's linear weights become 1x1 convolutions."""
    out = {}
    attn = {"group_norm": "norm", "to_q": "q", "to_k": "k", "to_v": "v", "to_out.0": "proj_out"}
    for k, v in sd.items():
        if not k.startswith("decoder."):
            continue
        r = k[len("decoder."):]
        if r.startswith("conv_norm_out."):
            nk = "norm_out." + r[len("conv_norm_out."):]
        elif r.startswith("mid_block.resnets."):
            i, rest = r[len("mid_block.resnets."):].split(".", 1)
            nk = f"mid.block_{int(i) + 1}.{rest}"
        elif r.startswith("mid_block.attentions.0."):
            rest = r[len("mid_block.attentions.0."):]
            name, leaf = rest.rsplit(".", 1)
            nk = f"mid.attn_1.{attn[name]}.{leaf}"
            if leaf == "weight" and name != "group_norm" and v.dim() == 2:
                v = v[:, :, None, None]
        elif r.startswith("up_blocks."):
            t, rest = r[len("up_blocks."):].split(".", 1)
            lvl = levels - 1 - int(t)
            if rest.startswith("resnets."):
                nk = f"up.{lvl}.block.{rest[len('resnets.'):]}"
            else:
                nk = f"up.{lvl}.upsample.conv.{rest[len('upsamplers.0.conv.'):]}"
        else:
            nk = r
        out["decoder." + nk.replace("conv_shortcut", "nin_shortcut")] = v
    return out


def convert_diffusers_vae_encoder(sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """AutoencoderKL encoder keys in diffusers naming -> the latent-diffusion naming of `OracleVaeEncoder`."""
    out = {}
    attn = {"group_norm": "norm", "to_q": "q", "to_k": "k", "to_v": "v", "to_out.0": "proj_out"}
    for k, v in sd.items():
        if not k.startswith("encoder."):
            continue
        r = k[len("encoder."):]
        if r.startswith("conv_norm_out."):
            nk = "norm_out." + r[len("conv_norm_out."):]
        elif r.startswith("mid_block.resnets."):
            i, rest = r[len("mid_block.resnets."):].split(".", 1)
            nk = f"mid.block_{int(i) + 1}.{rest}"
        elif r.startswith("mid_block.attentions.0."):
            name, leaf = r[len("mid_block.attentions.0."):].rsplit(".", 1)
            nk = f"mid.attn_1.{attn[name]}.{leaf}"
            if leaf == "weight" and name != "group_norm" and v.dim() == 2:
                v = v[:, :, None, None]
        elif r.startswith("down_blocks."):
            lvl, rest = r[len("down_blocks."):].split(".", 1)
            nk = f"down.{lvl}.block.{rest[len('resnets.'):]}" if rest.startswith("resnets.") else \
                f"down.{lvl}.downsample.conv.{rest[len('downsamplers.0.conv.'):]}"
        else:
            nk = r
        out["encoder." + nk.replace("conv_shortcut", "nin_shortcut")] = v
    return out


class T5OnlyEncoder:
    """T5 without padding: one row per prompt token plus the end-of-sequence token."""

    def __init__(self, t5, tokenizer):
        self.t5, self.tok = t5, tokenizer

    def encode(self, prompt: str) -> torch.Tensor:
        ids = self.tok.sp.encode(prompt) + [self.tok.eos]
        return self.t5.encode(torch.tensor([ids], dtype=torch.int64))


class HashT5:
    """Weight-free stand-in (synthetic snapshots): a fixed pseudo-random row per (byte pair, position)."""

    def __init__(self, dim: int, device, dtype):
        from .text_encoders import HashTextEncoders

        self.h = HashTextEncoders(dim, 8, device, dtype)

    def encode(self, prompt: str) -> torch.Tensor:
        n = max(1, len(prompt.encode("utf-8")))
        return self.h.encode(prompt, n).txt


@dataclass
class _Heavy:
    dit: Any
    vae: Any


class ChromaPipeline:
    def __init__(self, variant: ChromaVariant, root: Path, backend: str, device: torch.device):
        self.variant, self.root, self.backend, self.device = variant, Path(root), backend, device
        self.dit_cfg, self.vae_cfg, self.text_kind, self.random_init = ChromaConfig(), VaeConfig(), "t5", None
        cfg_path = self.root / "swb_config.json"
        if cfg_path.exists():
            raw = json.loads(cfg_path.read_text())
            if "dit" in raw:
                self.dit_cfg = ChromaConfig.from_json(raw["dit"])
            if "vae" in raw:
                v = dict(raw["vae"])
                if "ch_mult" in v:
                    v["ch_mult"] = tuple(v["ch_mult"])
                self.vae_cfg = VaeConfig(**v)
            self.text_kind = raw.get("text", self.text_kind)
            self.random_init = raw.get("random_init")
        elif (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = ChromaConfig.from_json(json.loads((self.root / "transformer" / "config.json").read_text()))
        self.dtype = torch.bfloat16 if backend == "b200" else torch.float32

    def load_text(self):
        if self.text_kind == "hash":
            return HashT5(self.dit_cfg.joint_attention_dim, self.device, self.dtype)
        from ..models.text_encoders import T5Config, T5Encoder
        from .text_models import T5SentencePieceTokenizer, _load_component

        for d in ("text_encoder", "tokenizer"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{self.variant.value}: snapshot {self.root} lacks {d}/")
        cfg, w = _load_component(self.root / "text_encoder")
        return T5OnlyEncoder(T5Encoder(T5Config.from_json(cfg), w, self.device, self.dtype),
                             T5SentencePieceTokenizer(self.root / "tokenizer" / "spiece.model"))

    def load_heavy(self) -> _Heavy:
        from ..io.safetensors_io import load_dir

        if self.random_init is not None and self.backend == "b200":
            from ..models.dit_chroma import ChromaDiTGpu
            from ..models.vae import VaeDecoderGpu

            seed = int(self.random_init)
            return _Heavy(ChromaDiTGpu(self.dit_cfg, device=self.device).init_random(seed),
                          VaeDecoderGpu(self.vae_cfg, self.device).init_random(seed + 1))
        for d in ("transformer", "vae"):
            if not (self.root / d).is_dir():
                raise LoadError(f"{self.variant.value}: snapshot {self.root} lacks {d}/")
        dit_w = load_dir(self.root / "transformer")
        vae_w = convert_diffusers_vae_decoder(load_dir(self.root / "vae"), len(self.vae_cfg.ch_mult))
        if self.backend == "b200":
            from ..models.dit_chroma import ChromaDiTGpu
            from ..models.vae import VaeDecoderGpu

            return _Heavy(ChromaDiTGpu(self.dit_cfg, device=self.device).load_state_dict(dit_w),
                          VaeDecoderGpu(self.vae_cfg, self.device).load_state_dict(vae_w))
        return _Heavy(OracleChromaDiT(self.dit_cfg, dit_w, device=self.device),
                      OracleVaeDecoder(self.vae_cfg, vae_w, device=self.device))

    def encode(self, text, req: GenerationRequest):
        guidance = req.true_cfg if req.true_cfg is not None else self.variant.default_true_cfg
        pos = text.encode(req.prompt)
        neg = text.encode(req.negative_prompt or "") if guidance > 1.0 else None
        return pos, neg

    def render(self, heavy: _Heavy, cond, req: GenerationRequest, on_progress) -> list[Image]:
        v = self.variant
        steps = req.steps or v.default_steps
        guidance = req.true_cfg if req.true_cfg is not None else v.default_true_cfg
        base_seed = req.seed if req.seed is not None else default_seed()
        lh, lw = req.height // 8, req.width // 8
        dev, dt = self.device, self.dtype
        fc = self.dit_cfg.flux_config()
        sigmas = chroma_sigmas(v, steps)
        branches = []
        for emb in cond:
            if emb is None:
                continue
            txt = emb.to(dev, dt)
            txt_ids, img_ids = make_ids(lh // 2, lw // 2, txt.shape[1], dev)
            branches.append((txt, txt_ids, img_ids, rope_table(torch.cat([txt_ids, img_ids], 0), fc.axes_dim, fc.theta)))

        def velocity(x, sigma):
            tt = torch.full((1,), float(sigma), device=dev)
            outs = []
            for txt, txt_ids, img_ids, rope in branches:
                if self.backend == "b200":
                    o = heavy.dit.forward_graphed(x, img_ids, txt, txt_ids, tt, None, None, rope=rope)
                else:
                    o = heavy.dit.forward(x, img_ids, txt, txt_ids, tt, None, None)
                outs.append(o.float())
            if len(outs) == 1:
                return outs[0]
            pos, neg = outs
            return neg + (pos - neg) * guidance

        def one_image(seed: int) -> Image:
            x = patchify(seeded_noise_nchw(seed, self.vae_cfg.z_channels, lh, lw)).to(dev, dt).contiguous()
            for i in range(steps):
                if req.cancel.is_cancelled():
                    raise Canceled(f"{v.value}: cancelled at step {i}")
                vel = velocity(x, sigmas[i])
                x = (x.float() + vel * (sigmas[i + 1] - sigmas[i])).to(dt).contiguous()
                on_progress(ProgressStep(i + 1, steps))
            if req.cancel.is_cancelled():
                raise Canceled(f"{v.value}: cancelled before decode")
            on_progress(ProgressDecoding())
            z = unpatchify(x.float(), lh, lw)
            if self.backend == "b200":
                host = heavy.vae.decode_rgb8(z)[0].cpu()
            else:
                img = heavy.vae.decode(z)[0].permute(1, 2, 0)
                host = torch.round((img.clamp(-1, 1) + 1) * 127.5).to(torch.uint8).cpu()
            return Image(width=req.width, height=req.height, pixels=host.contiguous().numpy().tobytes())

        return for_each_image_seed(base_seed, req.count, one_image)


def chroma_descriptor(variant: ChromaVariant, backend: str, prefix: str = "") -> ModelDescriptor:
    """Only the wired surface is advertised: true CFG with a negative prompt; no adapters, quantised loading or
    control branches."""
    return ModelDescriptor(
        id=prefix + variant.value, family="chroma", backend=backend, modality=Modality.IMAGE,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=False, supports_true_cfg=True, conditioning=[],
            supports_lora=False, supports_lokr=False, samplers=["euler"] if "euler" in SOLVERS else list(SOLVERS)[:1],
            schedulers=[], supported_guidance_methods=[], min_size=256, max_size=2048, max_count=8,
            supports_sequential_offload=True),
        required_components=[])


class ChromaGenerator(Generator):
    def __init__(self, pipe: ChromaPipeline, descriptor: ModelDescriptor, policy: OffloadPolicy):
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
        if req.steps == 0:
            raise InferenceError(f"{mid}: steps must be >= 1 (an explicit 0 renders undenoised noise)")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} "
                                 f"(got {req.width}x{req.height})")

    def generate(self, req: GenerationRequest, on_progress: Callable = lambda p: None) -> GenerationOutput:
        self.validate(req)
        images = self.residency.run(req.cancel, on_progress, lambda text: self.pipe.encode(text, req),
                                    lambda heavy, cond: self.pipe.render(heavy, cond, req, on_progress))
        return GenerationOutput(images=images)


def _load(variant: ChromaVariant, backend: str, prefix: str) -> Callable[[LoadSpec], ChromaGenerator]:
    def load(spec: LoadSpec) -> ChromaGenerator:
        mid = prefix + variant.value
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
        return ChromaGenerator(ChromaPipeline(variant, Path(spec.weights.path), backend, device),
                               chroma_descriptor(variant, backend, prefix), spec.offload_policy)
    return load


def registrations(backend: str = "b200") -> list[Registration]:
    prefix = "" if backend == "b200" else "cpu_"
    return [Registration(descriptor=(lambda v=v: chroma_descriptor(v, backend, prefix)), load=_load(v, backend, prefix))
            for v in (ChromaVariant.HD, ChromaVariant.BASE, ChromaVariant.FLASH)]


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny random Chroma-shaped snapshot in the diffusers directory layout with the weight-free prompt encoder."""
    from ..io.safetensors_io import save_file
    from ..models.dit_chroma import random_chroma_weights
    from ..models.vae import random_vae_weights

    root = Path(root)
    dit = ChromaConfig(in_channels=64, num_layers=2, num_single_layers=2, attention_head_dim=128, num_attention_heads=2,
                       joint_attention_dim=64, approximator_num_channels=64, approximator_hidden_dim=128,
                       approximator_layers=2)
    vae = VaeConfig(ch=32, ch_mult=(1, 2, 2, 2), num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_chroma_weights(dit, seed).items()},
              root / "transformer" / "diffusion_pytorch_model.safetensors")
    native = random_vae_weights(vae, seed + 1)
    save_file({k: v.bfloat16() for k, v in native_vae_to_diffusers(native, len(vae.ch_mult)).items()},
              root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {k: (list(getattr(dit, k)) if k == "axes_dims_rope" else getattr(dit, k))
                for k in ChromaConfig.__dataclass_fields__},
        "vae": {"ch": vae.ch, "ch_mult": list(vae.ch_mult), "num_res_blocks": vae.num_res_blocks}, "text": "hash"}))
    return root


def native_vae_to_diffusers(sd: dict[str, torch.Tensor], levels: int = 4) -> dict[str, torch.Tensor]:
    """Inverse of convert_diffusers_vae_decoder (used to write synthetic diffusers-layout snapshots)."""
    out = {}
    attn = {"norm": "group_norm", "q": "to_q", "k": "to_k", "v": "to_v", "proj_out": "to_out.0"}
    for k, v in sd.items():
        r = k[len("decoder."):]
        if r.startswith("norm_out."):
            nk = "conv_norm_out." + r[len("norm_out."):]
        elif r.startswith("mid.block_"):
            i, rest = r[len("mid.block_"):].split(".", 1)
            nk = f"mid_block.resnets.{int(i) - 1}.{rest}"
        elif r.startswith("mid.attn_1."):
            name, leaf = r[len("mid.attn_1."):].rsplit(".", 1)
            nk = f"mid_block.attentions.0.{attn[name]}.{leaf}"
            if leaf == "weight" and name != "norm":
                v = v.reshape(v.shape[0], v.shape[1])
        elif r.startswith("up."):
            lvl, rest = r[len("up."):].split(".", 1)
            t = levels - 1 - int(lvl)
            nk = f"up_blocks.{t}.resnets.{rest[len('block.'):]}" if rest.startswith("block.") else \
                f"up_blocks.{t}.upsamplers.0.conv.{rest[len('upsample.conv.'):]}"
        else:
            nk = r
        out["decoder." + nk.replace("nin_shortcut", "conv_shortcut")] = v
    return out
