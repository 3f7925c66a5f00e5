"""One-process-per-GPU parallel runtime: bootstrap, NCCL baseline collectives, symmetric memory and the
fused compute+collective kernels (tensor parallel for the LLM engine, Ulysses sequence parallel for the DiT)."""
from .comm import Communicator, default_communicator, init_distributed, set_default_communicator, single  # noqa: F401
