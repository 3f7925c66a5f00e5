"""Continuous-batching serving benchmark: N concurrent requests with prompt lengths uniform in [lo, hi] random ids and a
fixed number of output tokens each, through `generate_continuous` (iteration-level batching over the paged KV cache)
on a tensor-parallel Llama decoder (torchrun: one rank per GPU). Reports aggregate generated tokens/s over the whole
job, decode-phase tokens/s, and p50 time to first token. --model 70b is Llama-3-70B (80 layers, hidden 8192, 64/8
heads, SwiGLU 28672); --model 8b the headline 8B; --layers overrides the depth for smoke runs (marks the line invalid)."""
import argparse
import json
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_config(name: str):
    from inference_b200.models import ModelConfig

    if name == "70b":
        return ModelConfig.from_json({
            "architectures": ["LlamaForCausalLM"], "hidden_size": 8192, "intermediate_size": 28672,
            "num_hidden_layers": 80, "num_attention_heads": 64, "num_key_value_heads": 8, "vocab_size": 128256,
            "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False,
            "max_position_embeddings": 8192})
    from bench import llama3_8b_config

    return llama3_8b_config()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="70b", choices=["70b", "8b"])
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--prompt-lo", type=int, default=256)
    ap.add_argument("--prompt-hi", type=int, default=4096)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--max-batch", type=int, default=128)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prefill-chunk", type=int, default=0,
                    help="> 0: at most this many prompt tokens per step, in the same forward as the decode rows")
    args = ap.parse_args()
    from inference_b200 import ops
    from inference_b200.engine.backend import GpuBackend
    from inference_b200.engine.decode import (BatchExactness, ContinuousConfig, ContinuousRequest,
                                              generate_continuous)
    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.parallel import init_distributed

    comm = init_distributed()
    cfg = model_config(args.model)
    invalid = None
    if args.layers:
        cfg.num_layers = args.layers
        invalid = f"smoke run with {args.layers} layers"
    if comm.world > 1 and os.environ.get("SWB_COMM", "auto") != "nccl":
        from inference_b200.parallel.symm import attach_fused

        attach_fused(comm)
    model = LlamaGpu(cfg, comm=comm, device=comm.device).init_random(seed=0)
    max_len = ((args.prompt_hi + args.new_tokens + 64 + 15) // 16) * 16
    eng = LlmEngine(model, EngineConfig(max_batch=args.max_batch, max_seq_len=max_len, prefill_token_budget=8192))
    backend = GpuBackend(eng.runner)
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(args.prompt_lo, args.prompt_hi + 1, (args.requests,), generator=g).tolist()
    reqs = [ContinuousRequest(torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist(), args.new_tokens)
            for n in lens]
    # warm-up: one short request per distinct graph shape is not possible (the batch shrinks only at the end), so
    # warm the kernels and allocator with a small job
    generate_continuous(backend, [ContinuousRequest(r.prompt[:64], 4) for r in reqs[:4]],
                        ContinuousConfig(max_batch=4, exactness=BatchExactness.THROUGHPUT))
    first = {}
    comm.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()

    def sink(i: int, tok: int) -> None:
        if i not in first:
            first[i] = time.perf_counter() - t0
    res = generate_continuous(backend, reqs, ContinuousConfig(max_batch=args.max_batch, prefill_chunk=args.prefill_chunk,
                                                              exactness=BatchExactness.THROUGHPUT), sink=sink)
    torch.cuda.synchronize()
    comm.barrier()
    total_s = comm.max_over_ranks(time.perf_counter() - t0)
    ops.check_status()
    generated = sum(len(r.tokens) for r in res)
    last_first = max(first.values())
    if comm.rank == 0:
        line = {"metric": "continuous_batching_tokens_per_s", "model": f"Llama-3-{args.model.upper()}",
                "n_gpus": comm.world, "parallelism": f"tp{comm.world}", "requests": args.requests,
                "prompt_tokens": sum(lens), "generated_tokens": generated, "total_s": round(total_s, 3),
                "value": round(generated / total_s, 1), "unit": "generated tokens/s (whole job, prefill included)",
                "decode_phase_tok_s": round((generated - args.requests) / max(1e-9, total_s - last_first), 1),
                "ttft_s_p50": round(statistics.median(first.values()), 3), "ttft_s_max": round(last_first, 3),
                "prefill_chunk": args.prefill_chunk, "dtype": "bf16", "data": "synthetic random ids, random-init weights",
                "kv_pool_gb": round(eng.pool.data.numel() * 2 / 1e9, 2)}
        if invalid:
            line["invalid"] = invalid
        print(json.dumps(line))
    comm.barrier()


if __name__ == "__main__":
    main()
