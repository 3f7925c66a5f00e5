"""Media engine: provider families built on the gen_core contracts (FLUX.1 text-to-image so far)."""
from .catalog import provider_registry  # noqa: F401
from .residency import Residency  # noqa: F401
from .seed import STEP_RNG_SALT, default_seed, for_each_image_seed, image_seed, seeded_noise_nchw  # noqa: F401
