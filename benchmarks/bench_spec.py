"""Speculative decoding benchmark: a Q4_K-quantised Llama-3-8B target with a Llama-3.2-1B-shaped bf16 draft, k = 4,
batch 1, 512-token prompt, 256 generated tokens (random-init weights, synthetic prompt). Reports tokens/s with and
without speculation, the measured acceptance rate and the verify-step latency (one target forward over k + 1
positions). With random weights the draft and target are unrelated, so the acceptance rate is the floor; --self-draft
uses the target as its own draft to show the ceiling of the mechanism."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--k", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--quant", default="Q4_K", help="Q4_K | Q8_0 | none")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--self-draft", action="store_true")
    args = ap.parse_args()
    from bench import llama3_8b_config
    from inference_b200 import ops
    from inference_b200.engine.backend import GpuBackend
    from inference_b200.engine.decode import (GenerationConfig, SpeculativeConfig, generate, generate_draft_speculative)
    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.parallel import init_distributed
    from inference_b200.policy import sampler as hs

    comm = init_distributed()
    dev = comm.device
    tcfg = llama3_8b_config()
    tcfg.num_layers = args.layers
    target = LlamaGpu(tcfg, comm=comm, device=dev).init_random(seed=0)
    dense_bytes = target.weight_bytes()
    if args.quant != "none":
        t0 = time.time()
        target.quantize_(args.quant)
        torch.cuda.synchronize()
        quant_s = time.time() - t0
    else:
        quant_s = 0.0
    dcfg = llama3_8b_config()
    dcfg.num_layers, dcfg.hidden_size, dcfg.intermediate_size = 16, 2048, 8192
    dcfg.num_heads, dcfg.num_kv_heads = 16, 4          # head_dim stays 128 (the kernels' head size)
    draft = target if args.self_draft else LlamaGpu(dcfg, comm=comm, device=dev).init_random(seed=1)
    L = args.prompt_len + args.new_tokens + 64
    ecfg = EngineConfig(max_batch=2, max_seq_len=L, prefill_token_budget=4096)
    tb = GpuBackend(LlmEngine(target, ecfg).runner)
    db = GpuBackend(LlmEngine(draft, ecfg).runner)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, tcfg.vocab_size, (args.prompt_len,), generator=g).tolist()
    gcfg = GenerationConfig(max_new_tokens=args.new_tokens, sampling=hs.SamplingParams(temperature=0.0))

    def timed(fn):
        fn()                                    # warm-up: graph captures, allocator
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = fn()
        torch.cuda.synchronize()
        return out, time.perf_counter() - t0

    base, base_s = timed(lambda: generate(tb, prompt, gcfg))
    (spec_res, stats), spec_s = timed(lambda: generate_draft_speculative(tb, db, prompt, gcfg,
                                                                         SpeculativeConfig(num_draft=args.k)))
    # verify-step latency: one target forward over k + 1 new positions on a 512-token context
    seq = tb.new_sequence()
    tb.forward([seq], [prompt])
    n = tb.length(seq)
    lat = []
    for _ in range(12):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tb.forward([seq], [prompt[: args.k + 1]], all_positions=True)
        e1.record()
        torch.cuda.synchronize()
        lat.append(e0.elapsed_time(e1))
        tb.truncate(seq, n)
    tb.release(seq)
    ops.check_status()
    lat.sort()
    print(json.dumps({
        "metric": "speculative_decode_tokens_per_s", "target": f"Llama-3-8B {args.layers}L {args.quant}",
        "draft": "self" if args.self_draft else "Llama-3.2-1B-shaped bf16 (16 layers, hidden 2048, 16/4 heads x 128)", "k": args.k, "prompt_len": args.prompt_len,
        "new_tokens": len(spec_res.tokens), "tokens_match_plain_greedy": spec_res.tokens == base.tokens,
        "plain_tok_s": round(len(base.tokens) / base_s, 1), "spec_tok_s": round(len(spec_res.tokens) / spec_s, 1),
        "acceptance_rate": round(stats.acceptance_rate, 4), "target_forwards": stats.forwards,
        "verify_ms_p50": round(lat[len(lat) // 2], 3), "weights_gb_dense": round(dense_bytes / 1e9, 2),
        "weights_gb_now": round(target.weight_bytes() / 1e9, 2), "quantize_s": round(quant_s, 1)}))


if __name__ == "__main__":
    main()
