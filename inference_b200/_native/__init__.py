"""ctypes loaders for the in-tree native libraries.

`kernels()` returns the sm_100a CUDA kernel library, `host()` the C++ host-policy library. Both are
built by `inference_b200/_native/build.py`; a missing library is an error (there is no silent PyTorch
fallback for a kernel on a GPU box).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_DIR = Path(__file__).resolve().parent
_KERNELS = None
_HOST = None


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str, builder: str):
    path = _DIR / name
    if not path.exists():
        if os.environ.get("SWB_NO_AUTOBUILD"):
            raise NativeLibraryMissing(f"{path} is missing; run `python -m inference_b200._native.build`")
        from . import build as _build

        getattr(_build, builder)()
    if not path.exists():
        raise NativeLibraryMissing(f"{path} could not be built")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def kernels() -> ctypes.CDLL:
    global _KERNELS
    if _KERNELS is None:
        _KERNELS = _load("libswb200_kernels.so", "build_kernels")
        _declare_kernels(_KERNELS)
    return _KERNELS


def host() -> ctypes.CDLL:
    global _HOST
    if _HOST is None:
        _HOST = _load("libswb200_host.so", "build_host")
    return _HOST


c_int = ctypes.c_int
c_void_p = ctypes.c_void_p
c_size_t = ctypes.c_size_t
c_float = ctypes.c_float
c_ll = ctypes.c_longlong


def _declare_kernels(lib: ctypes.CDLL) -> None:
    def sig(name, argtypes, restype=c_int):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = restype

    sig("swb_status_read", [ctypes.POINTER(c_int)])
    sig("swb_status_clear", [])
    sig("swb_set_wait_limit_ns", [ctypes.c_ulonglong])
    sig("swb_set_timeline", [c_void_p])
    sig("swb_gemm_set_trace", [c_void_p], None)
    sig("swb_sm_count", [])
    sig("swb_gemm_workspace_min", [], c_size_t)
    sig("swb_gemm_bf16", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_void_p, c_size_t, c_int, c_int, c_int, c_void_p])
    sig("swb_rmsnorm_prefetch", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                 c_float, c_void_p, c_ll, c_void_p])
    sig("swb_rmsnorm", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float,
                        c_void_p])
    sig("swb_layernorm_mod", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                              c_int, c_int, c_float, c_void_p])
    sig("swb_rope_kv_write", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                              c_void_p, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                              c_void_p])
    sig("swb_gated_act_mul", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    sig("swb_embedding", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p])
    sig("swb_gated_residual", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p])
    sig("swb_attn_decode_workspace_bytes", [c_int, c_int, c_int], c_size_t)
    sig("swb_attn_paged", [c_void_p, c_ll, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int,
                           c_int, c_void_p, c_size_t, c_void_p])
    sig("swb_attn_dense", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_ll, c_int, c_int,
                           c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    sig("swb_axpy", [c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_int, c_void_p])
    sig("swb_groupnorm", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
                          c_void_p])
    sig("swb_upsample2x", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    sig("swb_attn_dense_set_impl", [c_int], None)
    sig("swb_attn_dense_set_tiles", [c_int], None)
    sig("swb_attn_varlen_causal", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_ll, c_void_p, c_int,
                                   c_int, c_int, c_int, c_int, c_float, c_void_p])
    sig("swb_attn_paged_prefill_tc", [c_void_p, c_ll, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    sig("swb_attn_dense_scatter", [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int, c_void_p, c_int,
                                   c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                   c_void_p])
    sig("swb_gemm_bf16_scatter", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_void_p])
    sig("swb_gemm_bf16_scatter_rows", [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                       c_int, c_void_p])
    sig("swb_nvfp4_quantize", [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                               c_void_p])
    sig("swb_nvfp4_quantize_fast", [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    sig("swb_dequant_nvfp4", [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p])
    sig("swb_gemm_nvfp4", [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                           c_void_p, ctypes.c_size_t, c_int, c_void_p])
    sig("swb_gemm_nvfp4_w4a4", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                                c_void_p, c_void_p])
    sig("swb_sample_device", [c_void_p, c_int, c_ll, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p])
    sig("swb_argmax_peer_merge", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    sig("swb_gemm_bf16_normed", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                 c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p])
    sig("swb_gemm_gated_supported", [c_int, c_int, c_int])
    sig("swb_gemm_bf16_peer_reduce", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_void_p])
    sig("swb_gemm_peer_max_ctas", [])
    sig("swb_decode_meta_unpack", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p])
    sig("swb_decode_step_tail", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    sig("swb_gemm_bf16_grouped", [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, c_void_p])
    sig("swb_reduce_norm_gather", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
    sig("swb_gemm_quant", [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p, ctypes.c_size_t, c_int, c_void_p])
    sig("swb_dequant_rows", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    sig("swb_peer_barrier", [c_void_p, c_void_p, c_int, c_int, c_void_p])
    sig("swb_im2col3x3", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    sig("swb_conv3x3_nhwc", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                             c_int, c_int, c_void_p])
    sig("swb_softmax_rows", [c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_float, c_void_p])
    sig("swb_rgb8", [c_void_p, c_void_p, c_ll, c_int, c_void_p])
    sig("swb_comm_max_ctas", [])
    sig("swb_comm_flag_words", [])
    sig("swb_allreduce_rmsnorm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_void_p, c_float, c_float, c_void_p, c_int, c_void_p])
    sig("swb_flag_wait", [c_void_p, ctypes.c_uint, c_void_p, c_void_p])
    sig("swb_set_pdl", [c_int], None)
    sig("swb_argmax", [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p])
    sig("swb_spec_verify_greedy", [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
    sig("swb_rep_penalty", [c_void_p, c_ll, c_int, c_int, c_void_p, c_int, c_void_p, c_float, c_void_p])
