"""Wan2.2 TI2V-5B text-to-video `wan2_2_ti2v_5b` (parity: candle-gen-wan/src/lib.rs, config.rs, vae.rs).

The dense 5B member of the family: one DiT (30 layers, width 3072, 24 heads of 128, 48-channel latents) instead of the
two 14B experts, and the z48 residual autoencoder whose latents are 16x smaller than the frame in each spatial direction
(4x in time). Classifier-free guidance 5 with the family's default negative prompt, flow shift 5, 40 UniPC (or Euler)
steps, 24 fps; sizes are multiples of 32 from 480 up to a 1280 x 704 frame area. LoRA / LoKr files are folded into the
DiT weights at load. Text-to-video only: image conditioning is not part of this provider."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..contracts.errors import InferenceError, LoadError, Unsupported
from ..contracts.gen_core.generator import Capabilities, GenerationRequest, Modality, ModelDescriptor
from ..contracts.gen_core.registry import Registration
from ..contracts.gen_core.runtime import AdapterKind, LoadSpec
from ..contracts.gen_core.sampling import SOLVERS
from ..contracts.gen_core.traits import reject_unknown_components
from ..models.dit_wan import WanConfig, WanDiT, random_wan_weights
from ..models.vae_qwen import Wan22VaeConfig, Wan22VaeDecoder, random_wan22_vae_weights
from .wan import WanGenerator, WanPipeline, WanVariant, _Heavy

MODEL_ID = "wan2_2_ti2v_5b"
DEFAULT_GUIDANCE, FLOW_SHIFT, DEFAULT_FPS, SIZE_MULTIPLE, MIN_SIZE, MAX_AREA_5B = 5.0, 5.0, 24, 32, 480, 1280 * 704
TI2V_5B = WanVariant(MODEL_ID, 0.0, FLOW_SHIFT, DEFAULT_GUIDANCE, DEFAULT_GUIDANCE, stride=16, fps=DEFAULT_FPS)


def ti2v_dit_config() -> WanConfig:
    return WanConfig(num_attention_heads=24, attention_head_dim=128, num_layers=30, ffn_dim=14336, in_channels=48, out_channels=48)


class WanTi2vPipeline(WanPipeline):
    def __init__(self, root: Path, backend: str, device: torch.device):
        super().__init__(root, backend, device, TI2V_5B)
        self.adapters: list = []
        raw = json.loads((self.root / "swb_config.json").read_text()) if (self.root / "swb_config.json").exists() else {}
        if "dit" not in raw and not (self.root / "transformer" / "config.json").exists():
            self.dit_cfg = ti2v_dit_config()
        self.vae22_cfg = Wan22VaeConfig(**raw["vae22"]) if "vae22" in raw else Wan22VaeConfig()
        if self.dit_cfg.out_channels != self.vae22_cfg.z_dim:
            raise LoadError(f"{MODEL_ID}: the DiT emits {self.dit_cfg.out_channels} channels but the autoencoder has "
                            f"{self.vae22_cfg.z_dim}")

    def load_heavy(self):
        from ..io.safetensors_io import load_dir
        from .family import fold_adapters

        if self.random_init is not None and self.backend == "b200":
            seed = int(self.random_init)
            dit_w = random_wan_weights(self.dit_cfg, seed, 0.02, torch.bfloat16, self.device)
            vae_w = random_wan22_vae_weights(self.vae22_cfg, seed + 2)
        else:
            for d in ("transformer", "vae"):
                if not (self.root / d).is_dir():
                    raise LoadError(f"{MODEL_ID}: snapshot {self.root} lacks {d}/")
            dit_w, vae_w = load_dir(self.root / "transformer"), load_dir(self.root / "vae")
            if self.adapters:
                dit_w = fold_adapters(dit_w, self.adapters, MODEL_ID)
        dit = WanDiT(self.dit_cfg, dit_w, self.dtype, self.device)
        return _Heavy(dit, dit, Wan22VaeDecoder(self.vae22_cfg, vae_w, torch.float32, self.device))


def ti2v_descriptor(backend: str, prefix: str = "") -> ModelDescriptor:
    return ModelDescriptor(
        id=prefix + MODEL_ID, family="wan", backend=backend, modality=Modality.VIDEO,
        capabilities=Capabilities(
            supports_negative_prompt=True, supports_guidance=True, supports_true_cfg=False, conditioning=[],
            supports_lora=True, supports_lokr=True, samplers=list(SOLVERS), schedulers=[], supported_guidance_methods=[],
            min_size=MIN_SIZE, max_size=1280, max_count=1, supports_sequential_offload=True),
        required_components=[])


class WanTi2vGenerator(WanGenerator):
    def validate(self, req: GenerationRequest) -> None:
        mid = self._descriptor.id
        self._descriptor.capabilities.validate_request(mid, req)
        if not req.prompt:
            raise InferenceError(f"{mid}: prompt must not be empty")
        if req.width % SIZE_MULTIPLE or req.height % SIZE_MULTIPLE:
            raise InferenceError(f"{mid}: width/height must be multiples of {SIZE_MULTIPLE} (got {req.width}x{req.height})")
        if req.frames is not None and (req.frames < 1 or (req.frames - 1) % 4):
            raise InferenceError(f"{mid}: frames must be 4k + 1 (got {req.frames})")
        if req.width * req.height > MAX_AREA_5B:
            raise InferenceError(f"{mid}: {req.width}x{req.height} exceeds the {MAX_AREA_5B}-pixel frame budget (1280 x 704)")
        if req.conditioning:
            raise InferenceError(f"{mid}: image / control conditioning is not supported (text-to-video only)")


def registration(backend: str = "b200") -> Registration:
    prefix = "" if backend == "b200" else "cpu_"

    def load(spec: LoadSpec) -> WanTi2vGenerator:
        mid = prefix + MODEL_ID
        if spec.weights is None or spec.weights.is_file:
            raise Unsupported(f"{mid}: needs a snapshot directory")
        if spec.quantize is not None:
            raise Unsupported(f"{mid}: quantised loading ({spec.quantize.name}) is not supported")
        reject_unknown_components(spec.components, [], mid)
        if spec.control or spec.extra_controls or spec.ip_adapter:
            raise Unsupported(f"{mid}: control branches and IP adapters are not supported by this provider")
        for ad in spec.adapters:
            if ad.kind not in (AdapterKind.LORA, AdapterKind.LOKR):
                raise Unsupported(f"{mid}: adapter kind {ad.kind.value} is not supported")
        if backend == "b200":
            if not torch.cuda.is_available():
                raise LoadError(f"{mid}: no CUDA device")
            device = torch.device("cuda", torch.cuda.current_device())
        else:
            device = torch.device("cpu")
        pipe = WanTi2vPipeline(Path(spec.weights.path), backend, device)
        pipe.adapters = list(spec.adapters)
        return WanTi2vGenerator(pipe, ti2v_descriptor(backend, prefix), spec.offload_policy)

    return Registration(descriptor=lambda: ti2v_descriptor(backend, prefix), load=load)


def write_synthetic_snapshot(root, seed: int = 0) -> Path:
    """A tiny one-expert snapshot: 2-layer DiT over 8-channel latents, a z8 residual autoencoder of base width 8."""
    from ..io.safetensors_io import save_file

    root = Path(root)
    dit = WanConfig(num_attention_heads=2, attention_head_dim=128, num_layers=2, ffn_dim=256, text_dim=64, in_channels=8, out_channels=8)
    vae = Wan22VaeConfig(z_dim=8, base_dim=8, num_res_blocks=1)
    (root / "transformer").mkdir(parents=True, exist_ok=True)
    (root / "vae").mkdir(exist_ok=True)
    save_file({k: v.bfloat16() for k, v in random_wan_weights(dit, seed, 0.05).items()}, root / "transformer" / "diffusion_pytorch_model.safetensors")
    save_file({k: v.bfloat16() for k, v in random_wan22_vae_weights(vae, seed + 2).items()}, root / "vae" / "diffusion_pytorch_model.safetensors")
    (root / "swb_config.json").write_text(json.dumps({
        "dit": {"num_attention_heads": 2, "attention_head_dim": 128, "num_layers": 2, "ffn_dim": 256, "text_dim": 64, "in_channels": 8,
                "out_channels": 8},
        "vae22": {"z_dim": 8, "base_dim": 8, "num_res_blocks": 1}, "text": "hash"}))
    return root
