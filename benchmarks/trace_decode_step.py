"""Per-kernel breakdown of ONE Llama-3-8B decode step replayed from its CUDA graph, from the in-kernel launch
timeline (`utils.tracing.LaunchTimeline`): for every launch the moment its predecessor had completely finished, so the
differences are each kernel's share of the critical path with programmatic dependent launch in effect. No profiler.

  python benchmarks/trace_decode_step.py                      # TP = 1
  python benchmarks/trace_decode_step.py --emulate-tp 8       # one rank's TP = 8 shard shapes, no communication
  torchrun --nproc-per-node N benchmarks/trace_decode_step.py # real TP = N (rank 0 prints)
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--emulate-tp", type=int, default=0)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=3, help="timeline windows; the last one is reported")
    args = ap.parse_args()
    from bench import llama3_8b_config
    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.parallel import init_distributed
    from inference_b200.utils.tracing import LaunchTimeline

    comm = init_distributed()
    cfg = llama3_8b_config()
    cfg.num_layers = args.layers
    if args.emulate_tp > 1:
        P = args.emulate_tp
        cfg.num_heads //= P
        cfg.num_kv_heads //= P
        cfg.intermediate_size //= P
        cfg.vocab_size //= P
    if comm.world > 1:
        from inference_b200.parallel.symm import attach_fused

        attach_fused(comm)
    model = LlamaGpu(cfg, comm=comm, device=comm.device).init_random(seed=0)
    B, S = args.batch, args.prompt_len
    eng = LlmEngine(model, EngineConfig(max_batch=B, max_seq_len=S + 128, prefill_token_budget=8192))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (S,), generator=g).tolist() for _ in range(B)]
    seqs = [eng.new_sequence() for _ in range(B)]
    toks = eng.prefill_batch(seqs, prompts)
    out = eng.runner.decode_multi(seqs, toks, 8)        # captures the graph, warms up
    toks = out[-1].tolist()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    comm.barrier()
    e0.record()
    out = eng.runner.decode_multi(seqs, toks, 16)
    e1.record()
    torch.cuda.synchronize()
    plain_ms = comm.max_over_ranks(e0.elapsed_time(e1)) / 16
    toks = out[-1].tolist()
    recs = None
    for _ in range(args.steps):
        comm.barrier()
        with LaunchTimeline(8192) as tl:
            out = eng.runner.decode_multi(seqs, toks, 2)
        toks = out[-1].tolist()
        recs = tl.records()
    if comm.rank != 0:
        return
    # the second of the two replayed steps (the first starts from an idle GPU)
    metas = [i for i, r in enumerate(recs) if r["name"] == "decode_meta_unpack"]
    step = recs[metas[1]:] if len(metas) > 1 else recs
    total = sum(r["span_ns"] or 0 for r in step) / 1e3
    print(json.dumps({"what": "decode step launch timeline", "tp": comm.world, "emulate_tp": args.emulate_tp,
                      "batch": B, "context": S, "layers": args.layers, "ms_per_step_events_no_timeline": round(plain_ms, 4),
                      "step_us_with_timeline": round(total, 1), "launches": len(step)}))
    for row in LaunchTimeline.summarize(step):
        print(json.dumps(row))
    # one layer in launch order (layer 3: steady state)
    gemm_idx = [i for i, r in enumerate(step) if r["name"] == "gemm_decode_cluster"]
    if len(gemm_idx) >= 16:
        lo, hi = gemm_idx[12], gemm_idx[16]
        print("layer 3 in launch order (name grid head_start_us span_us):")
        for r in step[lo:hi]:
            print(f"  {r['name']:<22} {r['grid']:>4} {(r['released_ns'] - r['entered_ns']) / 1e3:7.2f} "
                  f"{(r['span_ns'] or 0) / 1e3:7.2f}")


if __name__ == "__main__":
    main()
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
