"""Decode-sized weight-only quantised GEMM on the Llama-3-8B projection shapes: time per call, effective packed-weight
bandwidth and the speed-up over the bf16 GEMM of the same shape (CUDA events, L2 flushed by rotating weight copies)."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters):
    """Microseconds per call with the calls replayed from one CUDA graph (no launch overhead between them)."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3   # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--formats", default="Q4_K,Q8_0,AFFINE4")
    args = ap.parse_args()
    from inference_b200 import ops
    from inference_b200.ops import quant

    T = args.tokens
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336)}
    rows = []
    for name, (N, K) in shapes.items():
        a = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
        base = torch.randn(N, K) * 0.02
        copies = max(2, (200 << 20) // (N * K // 2) + 1)
        dense = [base.bfloat16().cuda() for _ in range(min(copies, 6))]
        us_dense = timeit(lambda i: ops.gemm_bf16(a, dense[i % len(dense)]), args.iters)
        row = {"shape": name, "N": N, "K": K, "T": T, "bf16_us": round(us_dense, 2)}
        for fmt in args.formats.split(","):
            q0 = quant.quantize_weight(base, fmt).to("cuda")
            qs = [q0] + [quant.QuantWeight(fmt, q0.packed.clone(), N, K, q0.scales, q0.biases) for _ in range(copies - 1)]
            us = timeit(lambda i: quant.linear_quant(a, qs[i % len(qs)]), args.iters)
            row[fmt] = {"us": round(us, 2), "packed_gbs": round(q0.nbytes / us / 1e3, 1),
                        "speedup_vs_bf16": round(us_dense / us, 2)}
        ops.check_status()
        rows.append(row)
        print(json.dumps(row))


if __name__ == "__main__":
    main()
