"""64-wide-head dense attention on the tcgen05 kernel: native (one swizzle atom per tile) vs zero-padded to 128 vs the
framework's scaled-dot-product call, at the SD3.5-Large and SDXL shapes. CUDA events after warm-up, L2 flushed between
timed launches. Prints one JSON line per shape."""
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from inference_b200 import ops


def timed(fn, flush, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ms = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
    return sorted(ms)[len(ms) // 2]


def main():
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for name, B, Sq, Skv, H, D in (("flux joint 1024px (128-wide heads)", 1, 4608, 4608, 24, 128),
                                   ("sd3.5-large joint 1024px", 2, 4250, 4250, 38, 64), ("sdxl self 64x64", 2, 4096, 4096, 10, 64),
                                   ("sdxl self 32x32", 2, 1024, 1024, 20, 64), ("sdxl cross", 2, 4096, 77, 10, 64)):
        g = torch.Generator(device="cuda").manual_seed(0)
        q, k, v = (torch.randn(B, s, H, D, device="cuda", generator=g).bfloat16() for s in (Sq, Skv, Skv))
        scale = D ** -0.5
        ref = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                               v.transpose(1, 2).float()).transpose(1, 2).reshape(B, Sq, H * D)
        native = ops.dense_attention(q, k, v, scale=scale)
        err = float((native.float() - ref).abs().max())
        os.environ["SWB_NARROW_ATTN"] = "padded"
        t_pad = timed(lambda: ops.dense_attention_padded(q, k, v, scale=scale), flush)
        os.environ["SWB_NARROW_ATTN"] = "kernel"
        t_nat = timed(lambda: ops.dense_attention(q, k, v, scale=scale), flush)
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        t_lib = timed(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt), flush)
        flops = 4.0 * B * H * Sq * Skv * D
        print(json.dumps({"shape": name, "D": D, "B": B, "Sq": Sq, "Skv": Skv, "H": H, "max_abs_err": round(err, 4),
                          "native_ms": round(t_nat, 4), "padded_ms": round(t_pad, 4), "library_sdpa_ms": round(t_lib, 4),
                          "native_tflops": round(flops / t_nat / 1e9, 1)}))


if __name__ == "__main__":
    main()
