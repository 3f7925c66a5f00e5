"""Reference-guided generation (img2img) pieces shared by the flow-matching providers: where the run enters the sigma
table, how the request's reference is read, and the reference image -> clean latents encode
(parity: the `init_time_step` convention of candle-gen-sd3/src/pipeline.rs and candle-gen-z-image/src/pipeline.rs)."""
from __future__ import annotations

import torch

from ..contracts.errors import InferenceError, LoadError
from ..contracts.gen_core.generator import ConditioningKind, GenerationRequest
from ..contracts.gen_core.media import Image


def init_time_step(steps: int, strength: float | None) -> int:
    """max(1, floor(steps * strength)) for a strength in (0, 1], 0 (plain text-to-image) otherwise; a higher strength
    enters the schedule later and keeps more of the reference."""
    if strength is None or not strength > 0.0:
        return 0
    return max(1, min(steps - 1, int(steps * min(strength, 1.0)))) if steps > 1 else 0


def reference_of(req: GenerationRequest, label: str = "generator"):
    """(image, strength) of the request's single REFERENCE conditioning, or None."""
    refs = [c for c in req.conditioning if c.kind is ConditioningKind.REFERENCE]
    if not refs:
        return None
    if len(refs) > 1 or refs[0].image is None:
        raise InferenceError(f"{label}: exactly one reference image is supported")
    return refs[0].image, refs[0].strength


def encode_reference_image(vae_cfg, encoder_weights: dict[str, torch.Tensor], image: Image, width: int, height: int,
                           device, label: str = "generator") -> torch.Tensor:
    """Reference image (resized to the request's size with Lanczos) -> clean latents [1, z, h/8, w/8]: the
    autoencoder's mean, scaled; the encoder runs in fp32 and is built on demand from `encoder.*` tensors in the
    latent-diffusion naming."""
    import numpy as np

    from ..contracts.gen_core.imageops import resize
    from ..models.vae import OracleVaeEncoder

    if "encoder.conv_in.weight" not in encoder_weights:
        raise LoadError(f"{label}: the snapshot's autoencoder has no encoder, which a reference image needs")
    if (image.width, image.height) != (width, height):
        image = resize(image, width, height, "lanczos")
    px = torch.from_numpy(np.frombuffer(bytes(image.pixels), dtype=np.uint8).reshape(height, width, 3).copy())
    x = px.permute(2, 0, 1)[None].float() / 127.5 - 1.0
    enc = {k: v.float() for k, v in encoder_weights.items() if k.startswith(("encoder.", "quant_conv."))}
    return OracleVaeEncoder(vae_cfg, enc, device=device).encode(x).float()
