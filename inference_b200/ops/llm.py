"""Wrappers for the fused LLM glue kernels (norms, RoPE + KV write, gated activations, embedding)."""
from __future__ import annotations

import torch

from .._native import kernels
from .runtime import check, ptr, require_cuda, stream_ptr


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None, w_offset: float = 0.0, prefetch: torch.Tensor | None = None,
            prefetch_bytes: int = 0) -> torch.Tensor:
    """out = rmsnorm(x [+ residual]) * (w + w_offset); `residual` (if given) becomes x + residual in place.
    `prefetch`: weights of the kernel that consumes this norm; the first `prefetch_bytes` of them (all when 0) are
    requested into L2 while the norm runs.

    Semantics of the reference rms_norm (candle-llm/src/primitives/nn.rs:21-32): fp32 statistics over the
    last dimension. w_offset = 1 gives the Gemma "+1" convention."""
    require_cuda(x, w)
    x2 = x.reshape(-1, x.shape[-1])
    T, H = x2.shape
    assert x2.stride(1) == 1 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, H)
    r2 = residual.reshape(-1, H) if residual is not None else None
    if prefetch is not None:
        nb = prefetch.numel() * prefetch.element_size()
        nb = min(nb, prefetch_bytes) if prefetch_bytes > 0 else nb
        rc = kernels().swb_rmsnorm_prefetch(x2.data_ptr(), x2.stride(0), ptr(r2), r2.stride(0) if r2 is not None else 0,
                                            w.data_ptr(), o2.data_ptr(), o2.stride(0), T, H, eps, w_offset,
                                            prefetch.data_ptr(), nb, stream_ptr())
    else:
        rc = kernels().swb_rmsnorm(x2.data_ptr(), x2.stride(0), ptr(r2), r2.stride(0) if r2 is not None else 0,
                                   w.data_ptr(), o2.data_ptr(), o2.stride(0), T, H, eps, w_offset, stream_ptr())
    check(rc, "swb_rmsnorm")
    return out.reshape(x.shape)


def layernorm_mod(x: torch.Tensor, *, scale: torch.Tensor | None = None, shift: torch.Tensor | None = None,
                  rows_per_batch: int = 0, gamma: torch.Tensor | None = None, beta: torch.Tensor | None = None,
                  eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = LN(x) [* gamma + beta] * (1 + scale[b]) + shift[b] (adaLN modulation, one vector per batch)."""
    require_cuda(x)
    x2 = x.reshape(-1, x.shape[-1])
    T, H = x2.shape
    if out is None:
        out = torch.empty_like(x2)
    o2 = out.reshape(-1, H)
    ld_mod = 0
    for m in (scale, shift):
        if m is not None:
            assert m.dtype == torch.bfloat16 and m.stride(-1) == 1
            ld_mod = m.reshape(-1, H).stride(0) if m.numel() > H else H
            if m.dim() >= 2 and m.shape[0] > 1:
                ld_mod = m.stride(0)
    rc = kernels().swb_layernorm_mod(x2.data_ptr(), x2.stride(0), ptr(scale), ptr(shift), ld_mod, rows_per_batch,
                                     ptr(gamma), ptr(beta), o2.data_ptr(), o2.stride(0), T, H, eps, stream_ptr())
    check(rc, "swb_layernorm_mod")
    return out.reshape(x.shape)


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                  cos: torch.Tensor, sin: torch.Tensor, kcache: torch.Tensor | None, vcache: torch.Tensor | None,
                  n_heads: int, n_kv_heads: int, head_dim: int, *, rot_dim: int | None = None,
                  interleaved: bool = False, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                  norm_eps: float = 1e-6, norm_w_offset: float = 0.0, block_size: int = 16) -> None:
    """In place on qkv [T, (Hq + 2 Hkv) * D]: per-head q/k RMSNorm (optional), RoPE on q and k; k and v are
    also written to the paged cache [blocks, Hkv, block_size, D] at slot_mapping (int64; -1 = skip)."""
    require_cuda(qkv, positions, cos, sin)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and positions.dtype == torch.int32
    assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
    if slot_mapping is not None:
        assert slot_mapping.dtype == torch.int64
    rd = rot_dim if rot_dim is not None else head_dim
    assert cos.shape[-1] == rd // 2
    rc = kernels().swb_rope_kv_write(qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), ptr(slot_mapping),
                                     cos.data_ptr(), sin.data_ptr(), rd, 1 if interleaved else 0, ptr(q_norm),
                                     ptr(k_norm), norm_eps, norm_w_offset, ptr(kcache), ptr(vcache), block_size, T,
                                     n_heads, n_kv_heads, head_dim, stream_ptr())
    check(rc, "swb_rope_kv_write")


def gated_act_mul(gate_up: torch.Tensor, act: str = "silu", out: torch.Tensor | None = None,
                  paired: bool = False) -> torch.Tensor:
    """out[t, f] = act(gate_up[t, f]) * gate_up[t, F + f] (SwiGLU / GeGLU, candle-llm models/llama.rs:1386-1391).
    paired: the projection's rows are interleaved (gate_0, up_0, gate_1, ...), out[t, f] = act(gu[t, 2f]) * gu[t, 2f+1]."""
    require_cuda(gate_up)
    g2 = gate_up.reshape(-1, gate_up.shape[-1])
    T, F2 = g2.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gate_up.dtype, device=gate_up.device)
    rc = kernels().swb_gated_act_mul(g2.data_ptr(), g2.stride(0), out.data_ptr(), out.stride(0), T, F,
                                     (2 if act in ("gelu", "gelu_tanh") else 1) + (2 if paired else 0), stream_ptr())
    check(rc, "swb_gated_act_mul")
    return out.reshape(*gate_up.shape[:-1], F)


def embedding(ids: torch.Tensor, table: torch.Tensor, *, scale: float = 1.0, vocab_start: int = 0,
              out: torch.Tensor | None = None) -> torch.Tensor:
    require_cuda(ids, table)
    assert ids.dtype == torch.int64 and table.is_contiguous()
    flat = ids.reshape(-1)
    T, H = flat.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    rc = kernels().swb_embedding(flat.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, vocab_start,
                                 vocab_start + table.shape[0], scale, stream_ptr())
    check(rc, "swb_embedding")
    return out


def gated_residual(a: torch.Tensor, b: torch.Tensor, gate: torch.Tensor | None = None, rows_per_batch: int = 0,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """out = a + gate[batch] * b (DiT gated residual) or a + b."""
    require_cuda(a, b)
    H = a.shape[-1]
    a2, b2 = a.reshape(-1, H), b.reshape(-1, H)
    assert a2.is_contiguous() and b2.is_contiguous()
    if out is None:
        out = torch.empty_like(a2)
    ld_gate = 0
    if gate is not None:
        ld_gate = gate.stride(0) if gate.dim() >= 2 and gate.shape[0] > 1 else H
    rc = kernels().swb_gated_residual(a2.data_ptr(), b2.data_ptr(), ptr(gate), ld_gate, rows_per_batch,
                                      out.data_ptr(), a2.shape[0], H, stream_ptr())
    check(rc, "swb_gated_residual")
    return out.reshape(a.shape)


_ARGMAX_SCRATCH: dict[int, torch.Tensor] = {}


def _argmax_scratch(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _ARGMAX_SCRATCH.get(idx)
    if t is None:
        t = torch.empty(1 << 20, dtype=torch.uint8, device=device)
        _ARGMAX_SCRATCH[idx] = t
    return t


def argmax(logits: torch.Tensor, allow_mask: torch.Tensor | None = None, out: torch.Tensor | None = None,
           out_vals: torch.Tensor | None = None) -> torch.Tensor:
    """Row-wise argmax (ties -> lowest index) of fp32/bf16 logits; allow_mask: optional uint8 [V]; out_vals:
    optional fp32 [rows] receiving the maxima."""
    require_cuda(logits)
    l2 = logits.reshape(-1, logits.shape[-1])
    assert l2.stride(1) == 1 and l2.dtype in (torch.float32, torch.bfloat16)
    if out is None:
        out = torch.empty(l2.shape[0], dtype=torch.int64, device=logits.device)
    scratch = _argmax_scratch(logits.device)
    rc = kernels().swb_argmax(l2.data_ptr(), 1 if l2.dtype == torch.float32 else 0, l2.stride(0), l2.shape[0],
                              l2.shape[1], ptr(allow_mask), out.data_ptr(), ptr(out_vals), scratch.data_ptr(), scratch.numel(),
                              stream_ptr())
    check(rc, "swb_argmax")
    return out


def sample_device(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniforms: torch.Tensor,
                  allow_mask: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  out_prob: torch.Tensor | None = None) -> torch.Tensor:
    """Row-wise draw from softmax(logits / temperature) restricted to the top_k largest weights and the top_p nucleus
    (either limit off with top_k <= 0 / top_p >= 1), on the device. `uniforms`: fp32 [rows] in [0, 1), one per row.
    Returns int64 [rows]; `out_prob` (fp32 [rows]) receives the drawn token's probability within the kept set."""
    require_cuda(logits, uniforms)
    l2 = logits.reshape(-1, logits.shape[-1])
    assert l2.stride(1) == 1 and l2.dtype in (torch.float32, torch.bfloat16) and temperature > 0
    assert uniforms.dtype == torch.float32 and uniforms.numel() == l2.shape[0]
    if out is None:
        out = torch.empty(l2.shape[0], dtype=torch.int64, device=logits.device)
    rc = kernels().swb_sample_device(l2.data_ptr(), 1 if l2.dtype == torch.float32 else 0, l2.stride(0), l2.shape[0], l2.shape[1],
                                     float(temperature), int(top_k), float(top_p), uniforms.data_ptr(), ptr(allow_mask),
                                     out.data_ptr(), ptr(out_prob), stream_ptr())
    check(rc, "swb_sample_device")
    return out


def spec_verify_greedy(target_ids: torch.Tensor, draft: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """target_ids [S, k+1], draft [S, k] (int64) -> (n_accepted int32 [S], next_token int64 [S])."""
    require_cuda(target_ids, draft)
    S, k = draft.shape
    n_acc = torch.empty(S, dtype=torch.int32, device=draft.device)
    nxt = torch.empty(S, dtype=torch.int64, device=draft.device)
    rc = kernels().swb_spec_verify_greedy(target_ids.contiguous().data_ptr(), draft.contiguous().data_ptr(), k, S,
                                          n_acc.data_ptr(), nxt.data_ptr(), stream_ptr())
    check(rc, "swb_spec_verify_greedy")
    return n_acc, nxt
