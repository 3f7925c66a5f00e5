"""Model definitions: configuration dispatch, the fp32 CPU oracle and the sm_100a GPU models."""
from .config import Architecture, ModelConfig, RopeSpec, build_rope  # noqa: F401
