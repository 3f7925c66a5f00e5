"""Microbenchmark of the tcgen05 GEMM on the Llama-3-8B / FLUX projection shapes.

Times each shape with CUDA events after warm-up, rotating through enough distinct weight copies that
the operands of consecutive iterations exceed L2, and prints achieved TFLOP/s and GB/s next to the
measured peaks when MEASURED_PEAKS.json is present. `--torch` adds the library GEMM for comparison.
"""
import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from inference_b200 import ops


def bench(fn, iters, graph=False):
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        g.replay()
        en.record()
        torch.cuda.synchronize()
        return st.elapsed_time(en) / iters
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for i in range(iters):
        fn(i)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--torch", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shapes", default="llama")
    ap.add_argument("--mode", type=int, default=-1)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--graph", action="store_true", help="time a CUDA graph of the iterations (no launch overhead)")
    args = ap.parse_args()
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    shapes = []
    if args.shapes == "llama":
        for T in (1, 8, 64, 1024, 8192):
            for N, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
                shapes.append((T, N, K))
        shapes += [(1, 128256, 4096), (64, 128256, 4096)]
    elif args.shapes == "dit":
        for T in (4608,):
            for N, K in ((9216, 3072), (3072, 3072), (12288, 3072), (3072, 12288), (21504, 3072), (3072, 15360)):
                shapes.append((T, N, K))
    else:
        for s in args.shapes.split(";"):
            shapes.append(tuple(int(x) for x in s.replace("x", ",").split(",")))
    rows = []
    for T, N, K in shapes:
        wbytes = N * K * 2
        copies = max(2, min(16, (256 << 20) // wbytes + 1))
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
        a = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        ms = bench(lambda i: ops.gemm_bf16(a, ws[i % copies], out=out, mode=args.mode, block_n=args.block_n,
                                           ctas=args.ctas), args.iters, args.graph)
        ops.check_status()
        flops = 2.0 * T * N * K
        byts = (N * K + T * K + T * N) * 2
        row = {"T": T, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
               "gbs": round(byts / ms / 1e6, 1)}
        if peaks:
            row["frac_tflops_of_measured"] = round(row["tflops"] / peaks["bf16_tflops"], 3)
            row["frac_hbm_of_measured"] = round(row["gbs"] / peaks["hbm_gbs"], 3)
        if args.torch:
            ms_t = bench(lambda i: torch.matmul(a, ws[i % copies].t(), out=out), args.iters, args.graph)
            row["torch_ms"] = round(ms_t, 4)
        rows.append(row)
        print(json.dumps(row), flush=True)
        del ws
    return rows


if __name__ == "__main__":
    main()
