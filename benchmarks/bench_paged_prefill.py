"""Prefill attention on top of earlier context over the paged KV cache (prefix-cache hits, chunked prefill, speculative
verification): the tcgen05 kernel reading pages through TMA vs the mma.sync kernel, Llama-3-8B heads (32 query / 8
key-value, 128 wide), page size 16. CUDA events after warm-up, L2 flushed between timed launches. One JSON line per
shape; FLOPs count the causal triangle actually computed."""
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
    Hq, Hkv, D, bs = 32, 8, 128, 16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    scale = D ** -0.5
    for name, seqs, q_len, ctx in (("chunk 512 on 2048 context", 4, 512, 2048), ("chunk 2048 on 8192 context", 1, 2048, 8192),
                                   ("prefix hit: 256 new on 4096 cached", 8, 256, 4096), ("verify 8 on 2048 context", 16, 8, 2048),
                                   ("chunk 2048 on 32768 context", 1, 2048, 32768)):
        kv = ctx + q_len
        per = (kv + bs - 1) // bs
        blocks = seqs * per + 4
        g = torch.Generator(device="cuda").manual_seed(0)
        kc = torch.randn(blocks, Hkv, bs, D, device="cuda", generator=g).bfloat16()
        vc = torch.randn(blocks, Hkv, bs, D, device="cuda", generator=g).bfloat16()
        table = torch.randperm(blocks - 4, device="cuda", generator=g).to(torch.int32).view(seqs, per).contiguous()
        q = torch.randn(seqs * q_len, Hq, D, device="cuda", generator=g).bfloat16()
        cu = (torch.arange(seqs + 1, device="cuda") * q_len).to(torch.int32)
        kvl = torch.full((seqs,), kv, dtype=torch.int32, device="cuda")

        def run():
            return ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=q_len, scale=scale, causal=True)

        os.environ["SWB_PAGED_PREFILL"] = "legacy"
        ref = run().float()
        t_old = timed(run, flush)
        os.environ["SWB_PAGED_PREFILL"] = "tcgen05"
        err = float((run().float() - ref).abs().max())
        t_new = timed(run, flush)
        flops = 4.0 * seqs * Hq * D * (q_len * ctx + q_len * (q_len + 1) / 2)
        print(json.dumps({"shape": name, "seqs": seqs, "q_len": q_len, "context": ctx, "max_abs_diff_vs_mma_sync": round(err, 4),
                          "tcgen05_ms": round(t_new, 4), "mma_sync_ms": round(t_old, 4), "speedup": round(t_old / t_new, 2),
                          "tcgen05_tflops": round(flops / t_new / 1e9, 1), "mma_sync_tflops": round(flops / t_old / 1e9, 1)}))


if __name__ == "__main__":
    main()
