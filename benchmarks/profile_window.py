"""Small, self-terminating workloads for profiler captures. Each one runs its warm-up, then brackets a few launches
with cudaProfilerStart/Stop so that `ncu --profile-from-start off` sees only those.

  --what decode   one Llama-3-8B decode step (batch 64, 1024-token context) replayed from its CUDA graph
  --what dit      one FLUX-shaped DiT denoise step (1024x1024) at reduced depth (--depth / --depth-single)
  --what gemm     one tcgen05 GEMM, T x N x K from --shape (operands larger than L2 by default)
  --what cluster  one decode GEMM through the cluster split-K kernel (T=64, N=4096, K=14336)
  --what quant    one Q4_K dequant-GEMM (T from --shape "Tx..", N=28672, K=4096: the gate/up projection)
  --what attn     one split-KV decode attention launch (batch 64, 8 KV heads, context 2048)
  --what attn_dense one dense non-causal attention launch (S=4608, 24 heads)
  --what conv     one implicit-GEMM 3x3 convolution, 512 x 512 x 256 -> 256 channels (134 MB in, 134 MB out)
  --what paged_prefill  one prefill-attention launch over paged K / V: 2048 new tokens on 8192 of context, 32 / 8 heads
  --what vae      one FLUX-class VAE decode, 128 x 128 latents -> 1024 x 1024 (about 115 launches, 1.3 GB live)
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def window(fn, warmup=2, reps=1):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", required=True)
    ap.add_argument("--shape", default="8192x4096x4096")
    ap.add_argument("--depth", type=int, default=2)
    ap.add_argument("--depth-single", type=int, default=4)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--reps", type=int, default=1)
    args = ap.parse_args()
    from inference_b200 import ops

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    if args.what == "gemm" or args.what == "cluster":
        T, N, K = (64, 4096, 14336) if args.what == "cluster" else map(int, args.shape.split("x"))
        a = torch.randn(T, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def fn():
            flush.zero_()
            ops.gemm_bf16(a, w)
        window(fn, reps=args.reps)
    elif args.what == "quant":
        from inference_b200.ops import quant

        T, (N, K) = int(args.shape.split("x")[0]) if "x" in args.shape and args.shape != "8192x4096x4096" else 1, (28672, 4096)
        a = (torch.randn(T, K, device=dev, generator=g) * 0.5).bfloat16()
        qw = quant.quantize_weight(torch.randn(N, K) * 0.02, "Q4_K").to(dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def fn():
            flush.zero_()
            quant.linear_quant(a, qw)
        window(fn, reps=args.reps)
    elif args.what == "attn":
        B, Hq, Hkv, ctx, bs = 64, 32, 8, 2048, 16
        nblk = B * ctx // bs
        kc = torch.randn(nblk, Hkv, bs, 128, device=dev, generator=g).bfloat16()
        vc = torch.randn(nblk, Hkv, bs, 128, device=dev, generator=g).bfloat16()
        bt = torch.randperm(nblk, device=dev, generator=g).int().view(B, ctx // bs)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(B, Hq, 128, device=dev, generator=g).bfloat16()
        window(lambda: ops.paged_attention(q, kc, vc, bt, lens, cu_q=None, max_q_len=1, scale=128 ** -0.5, decode=True,
                                           num_splits=4), reps=args.reps)
    elif args.what == "attn_dense":
        S, H = 4608, 24
        q, k, v = (torch.randn(1, S, H, 128, device=dev, generator=g).bfloat16() for _ in range(3))
        window(lambda: ops.dense_attention(q, k, v, scale=128 ** -0.5, causal=False), reps=args.reps)
    elif args.what == "conv":
        x = torch.randn(1, 512, 512, 256, device=dev, generator=g).bfloat16()
        w = (torch.randn(256, 9 * 256, device=dev, generator=g) / 48).bfloat16()
        b = torch.randn(256, device=dev, generator=g).bfloat16()
        window(lambda: ops.conv3x3_nhwc(x, w, b), reps=args.reps)
    elif args.what == "paged_prefill":
        Hq, Hkv, D, bs, q_len, ctx = 32, 8, 128, 16, 2048, 8192
        per = (ctx + q_len) // bs
        kc = torch.randn(per + 4, Hkv, bs, D, device=dev, generator=g).bfloat16()
        vc = torch.randn(per + 4, Hkv, bs, D, device=dev, generator=g).bfloat16()
        table = torch.randperm(per, device=dev, generator=g).to(torch.int32).view(1, per).contiguous()
        q = torch.randn(q_len, Hq, D, device=dev, generator=g).bfloat16()
        cu = torch.tensor([0, q_len], dtype=torch.int32, device=dev)
        kvl = torch.tensor([ctx + q_len], dtype=torch.int32, device=dev)
        window(lambda: ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=q_len, scale=D ** -0.5, causal=True), reps=args.reps)
    elif args.what == "vae":
        from inference_b200.models.vae import VaeConfig, VaeDecoderGpu

        dec = VaeDecoderGpu(VaeConfig(), device=dev).init_random(0)
        z = torch.randn(1, 16, 128, 128, device=dev, generator=g)
        window(lambda: dec.decode(z), reps=args.reps)
    elif args.what == "dit":
        from inference_b200.contracts.gen_core.sampling import build_flow_sigmas, compute_mu, image_seq_len
        from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, make_ids, rope_table

        cfg = FluxConfig(depth=args.depth, depth_single=args.depth_single)
        model = FluxDiTGpu(cfg, device=dev).init_random(0)
        ht, St = 64, 512
        x = torch.randn(1, ht * ht, 64, device=dev, generator=g).bfloat16()
        txt = torch.randn(1, St, 4096, device=dev, generator=g).bfloat16()
        y = torch.randn(1, 768, device=dev, generator=g).bfloat16()
        txt_ids, img_ids = make_ids(ht, ht, St, dev)
        rope = rope_table(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.theta)
        gd = torch.full((1,), 3.5, device=dev)
        t = torch.full((1,), 0.7, device=dev)
        window(lambda: model.forward(x, img_ids, txt, txt_ids, t, y, gd, rope=rope), reps=args.reps)
    elif args.what == "decode":
        from bench import llama3_8b_config
        from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
        from inference_b200.models.llama import LlamaGpu
        from inference_b200.parallel import init_distributed

        comm = init_distributed()
        cfg = llama3_8b_config()
        cfg.num_layers = args.layers
        model = LlamaGpu(cfg, comm=comm, device=comm.device).init_random(seed=0)
        eng = LlmEngine(model, EngineConfig(max_batch=64, max_seq_len=1024 + 64, prefill_token_budget=8192))
        gen = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (1024,), generator=gen).tolist() for _ in range(64)]
        seqs = [eng.new_sequence() for _ in range(64)]
        toks = eng.prefill_batch(seqs, prompts)
        state = {"toks": toks}

        def fn():
            state["toks"] = eng.runner.decode_multi(seqs, state["toks"], 1)[-1].tolist()
        window(fn, warmup=3, reps=args.reps)
    else:
        raise SystemExit(f"unknown --what {args.what}")
    ops.check_status()
    print("ok", args.what)


if __name__ == "__main__":
    main()
