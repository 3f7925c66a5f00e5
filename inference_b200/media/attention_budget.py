"""Eager scaled-dot-product attention with a bound on the score matrix (candle-gen/src/attention.rs:40-153).

The reference chunks query rows so that B*H*Sq*Sk stays under 1e9 elements (its eager kernels index with 32-bit
integers). Here the fused tcgen05 attention never materialises scores, so this path is the CPU / oracle fallback
and the reference for chunked evaluation: chunks are independent, the result equals the single pass."""
from __future__ import annotations

import torch

ATTN_SCORES_BUDGET = 1_000_000_000


def query_block(rows_per_query: int, sq: int, budget: int) -> int:
    """Query rows per chunk: all of them when the whole score tensor fits, else budget / (score elements per row)."""
    if rows_per_query * sq <= budget:
        return sq
    return max(1, budget // max(1, rows_per_query))


def sdpa_budgeted_bhsd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                       mask: torch.Tensor | None = None, budget: int = ATTN_SCORES_BUDGET) -> torch.Tensor:
    """q [B,H,Sq,D], k / v [B,H,Sk,D]; mask broadcastable to [B,H,Sq,Sk] (additive)."""
    b, h, sq, _ = q.shape
    sk = k.shape[2]
    kt = k.transpose(2, 3)
    block = query_block(b * h * sk, sq, budget)
    outs = []
    for s in range(0, sq, block):
        n = min(block, sq - s)
        scores = (q[:, :, s:s + n] @ kt) * scale
        if mask is not None:
            scores = scores + (mask[:, :, s:s + n] if mask.shape[2] == sq else mask)
        outs.append(torch.softmax(scores.float(), dim=-1).to(v.dtype) @ v)
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=2)


def sdpa_budgeted_flat(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                       budget: int = ATTN_SCORES_BUDGET) -> torch.Tensor:
    """q / k / v [N, S, D] (batch and heads already merged)."""
    return sdpa_budgeted_bhsd(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), scale, None, budget).squeeze(0)
