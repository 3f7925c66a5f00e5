"""Python wrappers over the sm_100a kernel library (tensors in, tensors out, current CUDA stream)."""
from .attention import (dense_attention, dense_attention_padded, narrow_heads_on_kernel, paged_attention,  # noqa: F401
                        varlen_causal_attention)
from .gemm import SSQ_WORDS, ssq_buffer, ssq_values, gemm_bf16, gemm_bf16_grouped, gemm_bf16_normed, gated_fused, gemm_workspace, linear, linear_gated  # noqa: F401
from .llm import (argmax, sample_device, embedding, gated_act_mul, gated_residual, layernorm_mod, rmsnorm, rope_kv_write,  # noqa: F401
                  spec_verify_greedy)
from .runtime import KernelError, check_status, device_status  # noqa: F401
from .dit import axpy, conv3x3_nhwc, conv3x3_supported, groupnorm_nhwc, im2col3x3_nhwc, rgb8_nhwc, softmax_rows, upsample2x_nhwc  # noqa: E402,F401
from .quant import QuantWeight, dequantize, linear_any, linear_quant, quantize_weight  # noqa: E402,F401
