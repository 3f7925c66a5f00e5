"""The media provider catalog of one backend (parity: candle-gen-catalog's `provider_registry()`): an explicit list,
no global state and no import-time discovery."""
from __future__ import annotations

from ..contracts.gen_core.registry import ProviderRegistry, ProviderRegistryBuilder


def provider_registry(backend: str = "b200") -> ProviderRegistry:
    from . import anima, bernini, boogu, chroma, scail2, sensenova, wan_ti2v, wan_vace, flux, flux2, ideogram, kolors, mochi, krea, qwen_image, sana, sd3, sdxl, svd, wan, z_image

    b = ProviderRegistryBuilder()
    b.register_generators(flux.registrations(backend))
    b.register_generators(chroma.registrations(backend))
    b.register_generators(z_image.registrations(backend))
    b.register_generators(sd3.registrations(backend))
    b.register_generators(qwen_image.registrations(backend))
    b.register_generators(sdxl.registrations(backend))
    b.register_generators(kolors.registrations(backend))
    b.register_generators(wan.registrations(backend))
    b.register_generators([wan_ti2v.registration(backend)])
    b.register_generators([wan_vace.registration(backend)])
    b.register_generators([bernini.registration(backend)])
    b.register_generators([scail2.registration(backend)])
    b.register_generators(boogu.registrations(backend))
    b.register_generators(sensenova.registrations(backend))
    b.register_generators(krea.registrations(backend))
    b.register_generators(flux2.registrations(backend))
    b.register_generators(sana.registrations(backend))
    b.register_generators(ideogram.registrations(backend))
    b.register_generators(mochi.registrations(backend))
    b.register_generators(anima.registrations(backend))
    b.register_generators(svd.registrations(backend))
    from .train import trainer_registration

    b.register("trainer", trainer_registration(backend))
    from .train import z_image_trainer_registration

    b.register("trainer", z_image_trainer_registration(backend))
    from .train import sdxl_trainer_registration

    b.register("trainer", sdxl_trainer_registration(backend))
    from .train import krea_trainer_registration, wan_trainer_registration

    b.register("trainer", wan_trainer_registration(backend))
    b.register("trainer", krea_trainer_registration(backend))
    from . import vision_providers

    for kind, regs in vision_providers.registrations(backend).items():
        for r in regs:
            b.register(kind, r)
    from . import joycaption

    b.register("captioner", joycaption.registration(backend))
    return b.build()
