"""Dense attention microbenchmark (FLUX joint-attention shape by default): tcgen05 kernel vs the mma.sync kernel,
CUDA-event timed, rotating through enough q/k/v copies that consecutive iterations do not hit L2."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=4608)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    from inference_b200 import ops
    from inference_b200.ops.attention import set_dense_impl

    B, S, H = args.batch, args.seq, args.heads
    copies = max(2, (160 << 20) // (3 * B * S * H * 256) + 1)
    qkv = [torch.randn(B, S, 3, H, 128, device="cuda").bfloat16() for _ in range(copies)]
    out = torch.empty(B, S, H * 128, device="cuda", dtype=torch.bfloat16)
    flops = 4.0 * B * H * S * S * 128
    res = {}
    from inference_b200._native import kernels

    for name, legacy, tiles in (("tcgen05", False, 0), ("tcgen05_1tile", False, 1), ("tcgen05_2tile", False, 2),
                                ("mma_sync", True, 0)):
        set_dense_impl(legacy)
        kernels().swb_attn_dense_set_tiles(tiles)

        def run(i):
            t = qkv[i % copies]
            ops.dense_attention(t[:, :, 0], t[:, :, 1], t[:, :, 2], scale=128 ** -0.5, out=out)
        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.iters):
            run(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        res[name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}
    set_dense_impl(False)
    kernels().swb_attn_dense_set_tiles(0)
    ops.check_status()
    print(json.dumps({"shape": {"batch": B, "seq": S, "heads": H, "head_dim": 128}, **res}))


if __name__ == "__main__":
    main()
