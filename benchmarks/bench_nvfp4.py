"""NVFP4 W4A4 GEMM (tcgen05 kind::mxf4nvf4, block-scaled) against the bf16 tcgen05 GEMM on DiT projection shapes.

Times the FP4 GEMM alone (activations already packed) and with the activation quantiser in front, with CUDA events
after warm-up, rotating weight copies so that consecutive iterations do not reuse L2."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from inference_b200 import ops
from inference_b200._native import kernels
from inference_b200.ops import nvfp4 as nv
from inference_b200.ops.runtime import check, stream_ptr


def timed(fn, iters):
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for i in range(iters):
        fn(i)
    en.record()
    torch.cuda.synchronize()
    return st.elapsed_time(en) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--shapes", default="4608x9216x3072;4608x3072x3072;4608x12288x3072;4608x3072x12288;8192x4096x4096;8192x14336x4096")
    args = ap.parse_args()
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    for s in args.shapes.split(";"):
        T, N, K = (int(v) for v in s.split("x"))
        copies = max(2, min(8, (256 << 20) // (N * K // 2) + 1))
        dense = [(torch.randn(N, K, device="cuda") * 0.02) for _ in range(2)]
        wq = [nv.quantize_on_device(dense[i % 2]) for i in range(copies)]
        wb = [dense[i % 2].bfloat16() for i in range(2)]
        x = (torch.randn(T, K, device="cuda") * 0.5).bfloat16()
        aq, sfa, gs = nv.quantize_device_raw(x)
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)

        def fp4_only(i):
            w = wq[i % copies]
            check(kernels().swb_gemm_nvfp4_w4a4(aq.data_ptr(), sfa.data_ptr(), gs.data_ptr(), w.packed.data_ptr(), w.scales.data_ptr(),
                                                w.global_scale, out.data_ptr(), out.stride(0), T, N, K, None, stream_ptr()), "w4a4")

        ms_fp4 = timed(fp4_only, args.iters)
        ms_full = timed(lambda i: nv.gemm_w4a4(x, wq[i % copies]), args.iters)
        ms_bf16 = timed(lambda i: ops.gemm_bf16(x, wb[i % 2], out=out), args.iters)
        # the same quantise + GEMM sequence replayed from a CUDA graph: device time without the host's launch overhead
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(2):
                nv.gemm_w4a4(x, wq[i % copies])
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                nv.gemm_w4a4(x, wq[i])
        ms_graph = timed(lambda i: g.replay(), max(3, args.iters // 2)) / copies
        ops.check_status()
        flops = 2.0 * T * N * K
        row = {"T": T, "N": N, "K": K, "fp4_gemm_ms": round(ms_fp4, 4), "fp4_tflops": round(flops / ms_fp4 / 1e9, 1),
               "fp4_with_act_quant_ms": round(ms_full, 4), "fp4_with_act_quant_graph_ms": round(ms_graph, 4), "bf16_gemm_ms": round(ms_bf16, 4),
               "bf16_tflops": round(flops / ms_bf16 / 1e9, 1), "speedup_gemm": round(ms_bf16 / ms_fp4, 2),
               "speedup_with_quant_graph": round(ms_bf16 / ms_graph, 2)}
        if peaks:
            row["fp4_vs_measured_bf16_peak"] = round(row["fp4_tflops"] / peaks["bf16_tflops"], 2)
        print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
