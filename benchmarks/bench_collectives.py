"""Fused collectives against their library baselines (torchrun, one rank per GPU; CUDA events, max over ranks, calls
replayed from one CUDA graph so launch overhead is excluded):

  allreduce_rmsnorm   row-parallel partial sums -> all-reduce + residual add + RMSNorm in one peer-memory kernel
                      vs  NCCL all_reduce + the RMSNorm kernel
  gemm_rs_ag          prefill: row-parallel GEMM with scatter epilogue + reduce/norm/all-gather kernel + barrier
                      vs  GEMM + NCCL all_reduce + RMSNorm kernel

Roofline per call: max(FLOPs / measured GEMM peak, bytes crossing NVLink per rank / 770 GB/s)."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed_graph(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(iters):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3      # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from inference_b200 import ops
    from inference_b200.parallel import init_distributed
    from inference_b200.parallel.symm import FusedCollectives
    from inference_b200.parallel.tp_prefill import TpPrefillContext

    comm = init_distributed()
    dev, P, H = comm.device, comm.world, args.hidden
    peaks = {}
    pp = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pp):
        peaks = json.load(open(pp))
    gemm_peak = peaks.get("bf16_tflops_sustained", 1390.0) * 1e12
    link = 770e9
    fc = FusedCollectives(comm, H, max_tokens=256)
    w = (torch.rand(H, device=dev) + 0.5).bfloat16()
    rows = []
    for T in (1, 8, 64, 256):
        part = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        res = (torch.randn(T, H, device=dev) * 0.5).bfloat16()
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

        def fused():
            fc.begin_capture() if torch.cuda.is_current_stream_capturing() and not fc._capturing else None
            for _ in range(2):            # an even number of calls keeps the double buffering balanced under capture
                buf, i = fc.exchange_buffer(T)
                buf.copy_(part)
                fc._launch(i, T, res, w, 1e-5, 0.0, out)

        def nccl():
            for _ in range(2):
                t = part.clone()
                dist.all_reduce(t)
                ops.rmsnorm(t, w, 1e-5, residual=res)
        us_f = comm.max_over_ranks(timed_graph(fused, args.iters)) / 2
        fc._capturing = False
        us_n = comm.max_over_ranks(timed_graph(nccl, args.iters)) / 2
        nv_bytes = T * H * 2 * (P - 1)          # each rank pulls every peer's partial rows
        roof = nv_bytes / link * 1e6
        rows.append({"op": "allreduce_rmsnorm", "T": T, "H": H, "world": P, "fused_us": round(us_f, 2),
                     "nccl_us": round(us_n, 2), "roofline_us": round(roof, 3), "fused_frac_of_roofline": round(roof / us_f, 3)})
    ctx = TpPrefillContext(comm, H, 8192)
    K = 14336 // P
    wd = (torch.randn(H, K, device=dev) * 0.02).bfloat16()
    for T in (1024, 8192):
        a = (torch.randn(T, K, device=dev) * 0.5).bfloat16()
        lo, n = ctx.my_rows(T)
        res_l = (torch.randn(max(n, 1), H, device=dev) * 0.5).bfloat16()
        res_f = (torch.randn(T, H, device=dev) * 0.5).bfloat16()

        def fused2():
            ctx.gemm_scatter_rows(a, wd)
            ctx.reduce_norm_gather(T, res_l, w, 1e-5)

        def nccl2():
            y = ops.gemm_bf16(a, wd)
            dist.all_reduce(y)
            ops.rmsnorm(y, w, 1e-5, residual=res_f)
        us_f = comm.max_over_ranks(timed_graph(fused2, args.iters))
        us_n = comm.max_over_ranks(timed_graph(nccl2, args.iters))
        flops = 2.0 * T * H * K
        nv_bytes = T * H * 2 * (P - 1) / P * 2      # scatter of partial rows out + gather of normed rows out, per rank
        roof = max(flops / gemm_peak, nv_bytes / link) * 1e6
        rows.append({"op": "gemm_rs_ag (down proj shard)", "T": T, "H": H, "K": K, "world": P, "fused_us": round(us_f, 1),
                     "nccl_us": round(us_n, 1), "roofline_us": round(roof, 1), "fused_frac_of_roofline": round(roof / us_f, 3)})
    ops.check_status()
    if comm.rank == 0:
        for r in rows:
            print(json.dumps(r))
    comm.barrier()


if __name__ == "__main__":
    main()
