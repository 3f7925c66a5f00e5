"""Python wrappers over the sm_100a kernel library (tensors in, tensors out, current CUDA stream)."""
from .gemm import gemm_bf16, linear, gemm_workspace  # noqa: F401
from .runtime import check_status, device_status, KernelError  # noqa: F401
