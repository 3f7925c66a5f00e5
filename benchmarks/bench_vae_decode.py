"""FLUX-class VAE decode (16-channel latents 128 x 128 -> 1024 x 1024 RGB) and its 3x3 convolutions: the implicit-GEMM
convolution (nine TMA-shifted views, no patch matrix) vs patch gather + GEMM (SWB_CONV3X3=im2col). CUDA events after
warm-up, L2 flushed between timed runs. One JSON line for the decoder and one per convolution shape."""
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from inference_b200 import ops
from inference_b200.models.vae import VaeConfig, VaeDecoderGpu


def timed(fn, flush, iters=8):
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
    dec = VaeDecoderGpu(VaeConfig()).init_random(0)
    z = torch.randn(1, 16, 128, 128, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    out = {}
    for mode in ("im2col", "implicit"):
        os.environ["SWB_CONV3X3"] = mode
        img = dec.decode(z)
        out[mode] = (timed(lambda: dec.decode(z), flush), dec.launches, img.float())
    diff = float((out["implicit"][2] - out["im2col"][2]).abs().max())
    print(json.dumps({"what": "vae decode 128x128 latents -> 1024x1024", "implicit_ms": round(out["implicit"][0], 3),
                      "im2col_ms": round(out["im2col"][0], 3), "speedup": round(out["im2col"][0] / out["implicit"][0], 2),
                      "max_abs_diff_between_paths": round(diff, 4)}))
    g = torch.Generator(device="cuda").manual_seed(1)
    for H, C, Co in ((1024, 128, 128), (512, 256, 256), (512, 256, 128), (256, 512, 512), (128, 512, 512)):
        x = torch.randn(1, H, H, C, device="cuda", generator=g).bfloat16()
        w = (torch.randn(Co, 9 * C, device="cuda", generator=g) / (9 * C) ** 0.5).bfloat16()
        b = torch.randn(Co, device="cuda", generator=g).bfloat16()
        t = {}
        for mode in ("im2col", "implicit"):
            os.environ["SWB_CONV3X3"] = mode
            t[mode] = timed(lambda: ops.conv3x3_nhwc(x, w, b), flush)
        flops = 2.0 * H * H * 9 * C * Co
        print(json.dumps({"conv3x3": f"{H}x{H}x{C}->{Co}", "implicit_ms": round(t["implicit"], 4), "im2col_ms": round(t["im2col"], 4),
                          "speedup": round(t["im2col"] / t["implicit"], 2), "implicit_tflops": round(flops / t["implicit"] / 1e9, 1)}))


if __name__ == "__main__":
    main()
