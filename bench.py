"""Headline benchmark: Llama-3-8B bf16 decode throughput (+ p50 TTFT) on N B200 GPUs, tensor parallel TP=N.

Workload (the named configuration): Llama-3-8B architecture (32 layers, hidden 4096, 32/8 heads, head_dim
128, SwiGLU 14336, vocab 128256, RoPE theta 500000), random N(0, 0.02) weights, paged KV cache with
16-token blocks, prompts of 1024 uniform-random ids, greedy decode. A "step" is one decode iteration of
the whole batch (default batch 64 => 64 tokens per step).

  value   tokens/s over K decode steps, device-timed with CUDA events (max over ranks): the engine's
          multi-step path (sampled token fed back on device, one graph launch per step).
  e2e     the same metric through the public per-step API (`ModelRunner.decode`, what
          `LlmEngine.generate_batch` calls): every step copies that step's metadata host->device from
          pinned memory and reads the sampled tokens back to the host.
  extra   p50 time-to-first-token of a 1024-token prompt at batch 1, and decode tok/s at batch 1 and 8.

`--impl reference` reports why the reference (a Rust/Candle workspace) cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = ("reference is a Rust/Candle Cargo workspace: pip install of the reference tree fails (no "
                         "setup.py/pyproject.toml), no cargo/rustc in the image, git crate deps need network")


def llama3_8b_config():
    from inference_b200.models import ModelConfig

    return ModelConfig.from_json({
        "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "intermediate_size": 14336,
        "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "vocab_size": 128256,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": False,
        "max_position_embeddings": 8192})


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = f"/tmp/swb_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="debug only: run ONE rank's tensor-parallel shard shapes without communication (invalid run)")
    ap.add_argument("--no-extra", action="store_true", help="skip the TTFT / batch-1 / batch-8 side measurements")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch

    from inference_b200.engine.llm_engine import EngineConfig, LlmEngine
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.parallel import init_distributed

    comm = init_distributed()
    world = comm.world
    if world != args.gpus and int(os.environ.get("WORLD_SIZE", "1")) == 1 and args.gpus > 1:
        print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks"}))
        return 2
    dev = comm.device
    K, W, B, S = args.steps, max(3, args.warmup), args.batch, args.prompt_len
    cfg = llama3_8b_config()
    invalid = None
    if args.layers:
        cfg.num_layers = args.layers
        invalid = f"debug run with {args.layers} layers"
    if args.emulate_tp > 1:
        P = args.emulate_tp
        cfg.num_heads //= P
        cfg.num_kv_heads //= P
        cfg.intermediate_size //= P
        cfg.vocab_size //= P
        invalid = (invalid or "") + f" single-rank shard shapes of tp{P}"

    if world > 1 and os.environ.get("SWB_COMM", "auto") != "nccl":
        try:
            from inference_b200.parallel.symm import attach_fused

            attach_fused(comm)
        except ImportError:
            pass
    model = LlamaGpu(cfg, comm=comm, device=dev).init_random(seed=0)
    max_len = ((S + 2 * (K + W) + 80 + 15) // 16) * 16
    eng = LlmEngine(model, EngineConfig(max_batch=B, max_seq_len=max_len, prefill_token_budget=8192))
    runner = eng.runner
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (S,), generator=g).tolist() for _ in range(B)]

    def sync_all():
        comm.barrier()
        torch.cuda.synchronize()

    extra = {}
    # ---- p50 TTFT at batch 1 (prompt ids on the host -> first token on the host) -------------------
    if not args.no_extra:
        ttfts = []
        for i in range(6):
            s = eng.new_sequence()
            sync_all()
            t0 = time.perf_counter()
            tok = runner.prefill([s], [prompts[i % B]])
            _ = tok.tolist()
            t1 = time.perf_counter()
            if i > 0:
                ttfts.append((t1 - t0) * 1e3)
            s.release()
        extra["ttft_ms_p50_batch1"] = round(comm.max_over_ranks(statistics.median(ttfts)), 3)
        for b_small in (1, 8):
            seqs = [eng.new_sequence() for _ in range(b_small)]
            toks = eng.prefill_batch(seqs, prompts[:b_small])
            out = runner.decode_multi(seqs, toks, 3)
            toks = out[-1].tolist()
            n = min(64, K)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync_all()
            e0.record()
            out = runner.decode_multi(seqs, toks, n)
            e1.record()
            sync_all()
            ms = comm.max_over_ranks(e0.elapsed_time(e1))
            extra[f"decode_tok_s_batch{b_small}"] = round(b_small * n / ms * 1e3, 1)
            for s in seqs:
                s.release()

    # ---- main configuration: batch B ---------------------------------------------------------------
    seqs = [eng.new_sequence() for _ in range(B)]
    sync_all()
    t0 = time.perf_counter()
    toks = eng.prefill_batch(seqs, prompts)
    torch.cuda.synchronize()
    extra["prefill_ms_batch"] = round((time.perf_counter() - t0) * 1e3, 2)

    out = runner.decode_multi(seqs, toks, W)          # warm-up (captures the graph)
    toks = out[-1].tolist()
    sampler = ClockSampler(dev.index or 0)
    if comm.rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    out = runner.decode_multi(seqs, toks, K)          # EXACTLY K timed steps
    e1.record()
    sync_all()
    ms_total = comm.max_over_ranks(e0.elapsed_time(e1))
    launches = runner.launches_last
    toks = out[-1].tolist()
    ms_step = ms_total / K
    value = B * K / ms_total * 1e3

    # ---- end to end through the per-step public API --------------------------------------------------
    for _ in range(W):
        toks = runner.decode(seqs, toks).tolist()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(K):
        toks = runner.decode(seqs, toks).tolist()     # H2D metadata + graph + D2H tokens + sync, every step
    torch.cuda.synchronize()
    comm.barrier()
    e2e_s = comm.max_over_ranks(time.perf_counter() - t0)
    clocks = sampler.stop() if comm.rank == 0 else {}
    st = None
    try:
        from inference_b200 import ops

        st = ops.device_status()
    except Exception:
        pass

    if comm.rank == 0:
        line = {
            "metric": "llama3_8b_decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: uniform-random prompt ids, random-init N(0,0.02) weights",
            "config": {"model": "Llama-3-8B (32L, h4096, 32/8 heads, ffn 14336, vocab 128256)", "global_batch": B,
                       "seq_len": S, "decode_steps": K, "parallelism": f"tp{world}", "kv_block": 16,
                       "l2_policy": "inputs larger than L2 (16 GB of weights + KV streamed every step)",
                       "sampling": "greedy on device"},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                       "reasons": clocks.get("reasons", []), "samples": clocks.get("samples", 0)},
            "e2e": {"value": round(B * K / e2e_s, 1), "unit": "tokens/s", "ms_per_step": round(e2e_s / K * 1e3, 4),
                    "h2d_bytes_per_step": runner.h2d_bytes_last, "d2h_bytes_per_step": runner.d2h_bytes_last},
            "gpu_launches": launches, "impl": "ours", "extra": extra,
        }
        if st is not None:
            line["device_status"] = st[0]
        if invalid:
            line["invalid"] = invalid
        print(json.dumps(line))
    comm.barrier()
    return 0


if __name__ == "__main__":
    rc = main()
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    sys.exit(rc)
