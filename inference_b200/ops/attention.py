"""Paged and dense attention wrappers (head_dim 128)."""
from __future__ import annotations

import os

import torch

from .._native import kernels
from .runtime import check, ptr, require_cuda, stream_ptr

_DECODE_WS: dict[int, torch.Tensor] = {}


def decode_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _DECODE_WS.get(idx)
    if ws is None or ws.numel() < nbytes:
        # zeroed: the head of the buffer holds the split-KV ticket counters, which the kernels leave at zero
        ws = torch.zeros(max(nbytes, 16 << 20), dtype=torch.uint8, device=device)
        _DECODE_WS[idx] = ws
    return ws


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    kv_lens: torch.Tensor, *, cu_q: torch.Tensor | None, max_q_len: int, scale: float,
                    causal: bool = True, decode: bool = False, num_splits: int = 1, softcap: float = 0.0,
                    out: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                    use_tma: bool = True) -> torch.Tensor:
    """q: [T, Hq, 128] (any token/head strides, unit inner stride); caches [blocks, Hkv, block_size, 128];
    block_table int32 [num_seqs, max_blocks]; kv_lens int32 [num_seqs] (context length including the new
    tokens); cu_q int32 [num_seqs + 1] or None when every sequence has exactly max_q_len query tokens.
    Bottom-right aligned causal mask like the reference SDPA (candle-llm/src/primitives/attention.rs:154-186).
    Prefill (decode=False) with page sizes that divide 128 and no soft cap runs on the tcgen05 kernel, which reads the
    pages through TMA; SWB_PAGED_PREFILL=legacy keeps the mma.sync kernel (comparison runs)."""
    require_cuda(q, kcache, vcache, block_table, kv_lens)
    T, Hq, D = q.shape
    Hkv, bs = kcache.shape[1], kcache.shape[2]
    assert q.stride(2) == 1 and kcache.is_contiguous() and vcache.is_contiguous()
    assert block_table.dtype == torch.int32 and kv_lens.dtype == torch.int32 and block_table.stride(1) == 1
    num_seqs = kv_lens.numel()
    if out is None:
        out = torch.empty((T, Hq * D), dtype=q.dtype, device=q.device)
    if (not decode and D == 128 and softcap == 0.0 and use_tma and bs % 8 == 0 and 128 % bs == 0
            and os.environ.get("SWB_PAGED_PREFILL", "tcgen05") != "legacy"):
        if cu_q is None:
            cu_q = torch.arange(num_seqs + 1, dtype=torch.int32, device=q.device) * max_q_len
        rc = kernels().swb_attn_paged_prefill_tc(q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0),
                                                 kcache.data_ptr(), vcache.data_ptr(), block_table.data_ptr(),
                                                 block_table.stride(0), bs, kcache.shape[0], cu_q.data_ptr(),
                                                 kv_lens.data_ptr(), num_seqs, max_q_len, T, Hq, Hkv, scale,
                                                 1 if causal else 0, stream_ptr())
        if rc != -3:
            check(rc, "swb_attn_paged_prefill_tc")
            return out
    ws_ptr, ws_bytes = None, 0
    if decode and num_splits > 1:
        need = kernels().swb_attn_decode_workspace_bytes(num_seqs, Hkv, num_splits)
        if workspace is None:
            workspace = decode_workspace(q.device, need)
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel()
    rc = kernels().swb_attn_paged(q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0),
                                  kcache.data_ptr(), vcache.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                                  bs, kcache.shape[0] if use_tma else 0, ptr(cu_q), kv_lens.data_ptr(), num_seqs, max_q_len, Hq, Hkv, D, scale, softcap,
                                  1 if causal else 0, 1 if decode else 0, num_splits, ws_ptr, ws_bytes, stream_ptr())
    check(rc, "swb_attn_paged")
    return out


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float, causal: bool = False,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """q [B, Sq, Hq, D], k/v [B, Skv, Hkv, D] (k and v share strides), D = 128 or 64 -> out [B, Sq, Hq*D]. Both widths
    run on the tcgen05 kernel (64-wide heads: one swizzle atom per tile, half the shared memory and MMA work)."""
    require_cuda(q, k, v)
    B, Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    assert q.stride(3) == 1 and k.stride(3) == 1 and k.stride() == v.stride()
    assert q.stride(0) == Sq * q.stride(1) and k.stride(0) == Skv * k.stride(1)
    if out is None:
        out = torch.empty((B, Sq, Hq * D), dtype=q.dtype, device=q.device)
    rc = kernels().swb_attn_dense(q.data_ptr(), q.stride(1), q.stride(2), k.data_ptr(), v.data_ptr(), k.stride(1),
                                  k.stride(2), out.data_ptr(), out.stride(1), B, Sq, Skv, Hq, Hkv, D, scale,
                                  1 if causal else 0, stream_ptr())
    check(rc, "swb_attn_dense")
    return out


def narrow_heads_on_kernel() -> bool:
    """Heads narrower than 128 run on the tcgen05 kernel (64 natively, other widths zero-padded to 128) unless
    SWB_NARROW_ATTN=library selects the framework's scaled-dot-product call. SWB_NARROW_ATTN=padded forces the
    zero-padded path for 64-wide heads too (comparison runs)."""
    import os

    return os.environ.get("SWB_NARROW_ATTN", "kernel") != "library"


def dense_attention_padded(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float) -> torch.Tensor:
    """dense_attention for head widths below 128. 64 (SD3 / SDXL blocks) runs natively; other widths (72 in the Qwen3-VL
    tower, 120 in Boogu) are zero-padded to 128 per head, which changes neither q . k nor the first D output columns.
    q [B, Sq, H, D], k / v [B, Skv, Hkv, D] bf16 -> [B, Sq, H * D]."""
    import os

    B, Sq, H, D = q.shape
    if D == 128 or (D == 64 and os.environ.get("SWB_NARROW_ATTN", "kernel") != "padded"):
        return dense_attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=scale)
    assert D < 128
    pad = (0, 128 - D)
    qp, kp, vp = (torch.nn.functional.pad(t, pad).contiguous() for t in (q, k, v))
    out = dense_attention(qp, kp, vp, scale=scale)
    return out.view(B, Sq, H, 128)[..., :D].reshape(B, Sq, H * D)


def set_dense_impl(legacy: bool) -> None:
    """Comparison runs only: True forces the mma.sync kernel for dense attention, False restores the tcgen05 kernel."""
    kernels().swb_attn_dense_set_impl(1 if legacy else 0)


def varlen_causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, max_q_len: int, *,
                            scale: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal self-attention over a packed batch of fresh sequences on the tcgen05 kernel. q [T, Hq, 128], k / v
    [T, Hkv, 128] (views into one QKV buffer are fine), cu_q int32 [num_seqs + 1] -> out [T, Hq * 128]."""
    require_cuda(q, k, v, cu_q)
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    assert D == 128 and q.stride(2) == 1 and k.stride(2) == 1 and k.stride() == v.stride() and cu_q.dtype == torch.int32
    if out is None:
        out = torch.empty((T, Hq * D), dtype=q.dtype, device=q.device)
    rc = kernels().swb_attn_varlen_causal(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), v.data_ptr(), k.stride(0),
                                          k.stride(1), out.data_ptr(), out.stride(0), cu_q.data_ptr(), cu_q.numel() - 1,
                                          max_q_len, T, Hq, Hkv, scale, stream_ptr())
    check(rc, "swb_attn_varlen_causal")
    return out
