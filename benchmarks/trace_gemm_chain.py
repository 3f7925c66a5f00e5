"""Phase stamps of the decode GEMMs inside a programmatic-dependent-launch chain (CUDA graph of several layers'
qkv -> o -> gate_up -> down projections on Llama-3-8B shard shapes): for the last layer's four launches, the mean over
CTAs of each phase's time since the CTA's dependency resolved. Uses the kernels' own phase trace (`swb_gemm_set_trace`:
start, setup done, dependency satisfied, accumulator complete, partials delivered, cluster barrier passed, outputs
stored, end); no profiler.

  python benchmarks/trace_gemm_chain.py --tp 8 --tokens 64
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--layers", type=int, default=6)
    args = ap.parse_args()
    from inference_b200 import ops
    from inference_b200._native import kernels

    L = kernels()
    dev = torch.device("cuda")
    P, T, H = args.tp, args.tokens, 4096
    hq, hkv, ffn = 32 // P, 8 // P, 14336 // P
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*s):
        return (torch.randn(*s, device=dev, generator=g) * 0.02).bfloat16()

    layers = [dict(qkv=rnd((hq + 2 * hkv) * 128, H), o=rnd(H, hq * 128), gu=rnd(2 * ffn, H), down=rnd(H, ffn))
              for _ in range(args.layers)]
    res = rnd(T, H)
    attn = rnd(T, hq * 128)
    ssq = [ops.ssq_buffer(dev), ops.ssq_buffer(dev)]
    traces = [torch.zeros(512 * 16, dtype=torch.int64, device=dev) for _ in range(4)]

    def run(trace_last: bool):
        for li, w in enumerate(layers):
            last = trace_last and li == len(layers) - 1
            if last:
                L.swb_gemm_set_trace(traces[0].data_ptr())
            ops.gemm_bf16_normed(res, w["qkv"], ssq_in=ssq[1], norm_dim=H, eps=1e-5)
            if last:
                L.swb_gemm_set_trace(traces[1].data_ptr())
            ops.gemm_bf16_normed(attn, w["o"], out=res, residual=res, ssq_out=ssq[0], ssq_zero=ssq[1])
            if last:
                L.swb_gemm_set_trace(traces[2].data_ptr())
            act = ops.gemm_bf16_normed(res, w["gu"], act="swiglu_pairs", ssq_in=ssq[0], norm_dim=H, eps=1e-5)
            if last:
                L.swb_gemm_set_trace(traces[3].data_ptr())
            ops.gemm_bf16_normed(act, w["down"], out=res, residual=res, ssq_out=ssq[1], ssq_zero=ssq[0])
            if last:
                L.swb_gemm_set_trace(None)

    run(False)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run(True)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"tp_shapes": P, "tokens": T, "layers": args.layers,
                      "us_per_layer_4_gemms": round(e0.elapsed_time(e1) / 10 / args.layers * 1e3, 2)}))
    names = ["start", "setup", "dep", "acc", "deliv", "cbar", "stored", "end"]
    shapes = {"qkv": layers[0]["qkv"].shape, "o": layers[0]["o"].shape, "gate_up": layers[0]["gu"].shape,
              "down": layers[0]["down"].shape}
    prev_end = None
    for name, tr in zip(shapes, traces):
        full = tr.view(-1, 16).cpu()
        full = full[full[:, 0] > 0]
        t = full[:, :8]
        clk = full[:, 8:].double()
        dep = t[:, 2].clone()
        dep[dep == 0] = t[dep == 0, 1]
        first_dep = int(t[:, 2][t[:, 2] > 0].min()) if (t[:, 2] > 0).any() else int(t[:, 1].min())
        rel = (t - first_dep).float() / 1e3
        row = {"gemm": name, "shape": list(shapes[name]), "ctas": int(t.shape[0]),
               "head_start_us": round(float(-rel[:, 0].mean()), 2)}
        for i in (3, 4, 5, 6, 7):
            v = rel[:, i][t[:, i] > 0]
            if v.numel():
                row[names[i] + "_mean"] = round(float(v.mean()), 2)
                row[names[i] + "_max"] = round(float(v.max()), 2)
        # epilogue in SM clock cycles (mean over CTAs): accumulator -> delivered -> barrier -> first group summed ->
        # first group stored -> its sum of squares sent -> all groups stored
        cyc = lambda a, b: round(float((clk[:, b - 8] - clk[:, a - 8])[clk[:, b - 8] > 0].mean()), 0) if (clk[:, b - 8] > 0).any() else None  # noqa: E731
        row["cycles"] = {"acc_to_deliv": cyc(12, 13), "deliv_to_barrier": cyc(13, 8), "barrier_to_first_sum": cyc(8, 9),
                         "first_sum_to_store": cyc(9, 10), "store_to_ssq": cyc(10, 14), "barrier_to_all_stored": cyc(8, 11)}
        if prev_end is not None:
            row["since_prev_kernel_end_us"] = round((first_dep - prev_end) / 1e3, 2)
        prev_end = int(t[:, 7].max())
        print(json.dumps(row))


if __name__ == "__main__":
    main()
