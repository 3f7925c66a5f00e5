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

          + the DiT half of the headline (FLUX-shaped DiT 1024 x 1024 seconds per image at SP = N through the
          generator API), the library-collective arm (NCCL all-reduce + unfused norms) and the TP = N vs TP = 1
          token check.

`--impl reference` probes the machine for a Rust toolchain and reports why the reference (a Rust/Candle
workspace) cannot run here.
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


def probe_reference() -> dict:
    """Looks for what a build of the reference (a Cargo workspace) would need on this machine and, when a Rust
    toolchain is present, tries an offline build of its LLM crate under a time limit. Returns the JSON line."""
    import shutil

    found = {"cargo": shutil.which("cargo"), "rustc": shutil.which("rustc"),
             "pip_target": os.path.isdir(os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref"))
             and bool(os.listdir(os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")))}
    ref = os.environ.get("SWB_REFERENCE_DIR", "/root/reference")
    found["reference_tree"] = os.path.isfile(os.path.join(ref, "Cargo.toml"))
    found["vendored_crates"] = os.path.isdir(os.path.join(ref, "vendor", "crates")) or \
        os.path.isdir(os.path.expanduser("~/.cargo/registry"))
    why = REFERENCE_UNAVAILABLE
    if found["cargo"] and found["rustc"] and found["reference_tree"]:
        import tempfile

        work = tempfile.mkdtemp(prefix="swb_ref_")
        try:
            shutil.copytree(ref, os.path.join(work, "src"), symlinks=True)
            r = subprocess.run([found["cargo"], "build", "--release", "--offline", "-p", "candle-llm", "--features",
                                "cuda"], cwd=os.path.join(work, "src"), capture_output=True, text=True, timeout=900)
            tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or [""]
            why = f"cargo found, offline build of candle-llm exited {r.returncode}: {tail[0][:200]}"
            if r.returncode == 0:
                why = ("cargo built candle-llm offline, but the reference ships no bench binary for the named "
                       "configuration (its bench is a #[test] over real checkpoints: candle-llm/tests/bench.rs)")
        except Exception as e:  # noqa: BLE001
            why = f"cargo found, offline build failed: {type(e).__name__}: {str(e)[:160]}"
    return {"impl": "reference", "unavailable": why, "probe": found}


def dit_section(comm, dev, images: int = 2) -> dict:
    """FLUX-shaped DiT (19 + 38 blocks, hidden 3072, 24 heads x 128), 1024 x 1024, 4096 image + 512 text tokens,
    28 Euler flow-matching steps with guidance 3.5, VAE decode to RGB8 on the host, through the generator API
    (`catalog().media().load(...).generate(request)`); sequence parallel over all ranks of the job."""
    import tempfile

    import torch

    from inference_b200.bundles import runtime_b200
    from inference_b200.contracts.gen_core import GenerationRequest, LoadSpec

    d = tempfile.mkdtemp()
    with open(os.path.join(d, "swb_config.json"), "w") as f:
        json.dump({"text": "hash", "random_init": 0}, f)
    gen = runtime_b200.catalog().media().load("flux1_dev", LoadSpec.from_dir(d))
    gen.pipe.timings = {}
    req = lambda seed: GenerationRequest(prompt="a photo of a fox", width=1024, height=1024, steps=28, seed=seed,  # noqa: E731
                                         guidance=3.5)
    gen.generate(req(0), lambda e: None)           # loads the weights, captures the step graph
    torch.cuda.synchronize()
    e2e, step_ms, vae_ms, dev_total = [], [], [], []
    for i in range(images):
        comm.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = gen.generate(req(1 + i), lambda e: None)
        e2e.append(comm.max_over_ranks(time.perf_counter() - t0))      # image bytes are on the host
        assert len(out.images[0].pixels) == 1024 * 1024 * 3
        t = gen.pipe.timings
        steps = t["step_ms"]
        step_ms.append(comm.max_over_ranks(sum(steps[1:]) / max(1, len(steps) - 1)))   # mean over steps after step 0
        vae_ms.append(comm.max_over_ranks(t["vae_ms"]))
        dev_total.append(comm.max_over_ranks(sum(steps) + t["vae_ms"]))
    dit = gen.residency.heavy.dit if hasattr(gen.residency, "heavy") and gen.residency.heavy is not None else None
    res = {"dit_s_per_image": round(min(dev_total) / 1e3, 4), "dit_ms_per_step": round(min(step_ms), 3),
           "vae_decode_ms": round(min(vae_ms), 3), "dit_e2e_s_per_image": round(min(e2e), 4),
           "dit_parallelism": f"sp{comm.world}", "dit_images_timed": images,
           "dit_config": "FLUX.1-dev shape: 19 double + 38 single blocks, 4096 image + 512 text tokens, 28 Euler "
                         "steps, guidance 3.5, 16-channel VAE decode to 1024x1024x3 RGB8 on the host; random-init "
                         "weights, hash prompt encoder"}
    if dit is not None and comm.world > 1:
        res["dit_sp_path"] = os.environ.get("SWB_SP", "fused")
    del gen
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of exactly --steps steps; value = median")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--emulate-tp", type=int, default=0,
                    help="debug only: run ONE rank's tensor-parallel shard shapes without communication (invalid run)")
    ap.add_argument("--no-extra", action="store_true", help="skip the TTFT / batch-1 / batch-8 side measurements")
    ap.add_argument("--no-dit", action="store_true", help="skip the DiT 1024x1024 seconds-per-image section")
    ap.add_argument("--no-baseline", action="store_true", help="skip the library-collective (NCCL, unfused) arm")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps(probe_reference()))
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
    K, W, B, S, R = args.steps, max(3, args.warmup), args.batch, args.prompt_len, max(1, args.repeats)
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

    want_fused = world > 1 and os.environ.get("SWB_COMM", "auto") != "nccl"
    if want_fused:
        from inference_b200.parallel.symm import attach_fused

        attach_fused(comm)
    model = LlamaGpu(cfg, comm=comm, device=dev).init_random(seed=0)
    comm_path = "none" if world == 1 else ("fused" if comm.fused is not None else "nccl")
    if want_fused and comm.fused is None:
        # the peer-memory data plane did not come up: say so and fail instead of timing the library fallback
        if comm.rank == 0:
            print(json.dumps({"error": "fused peer-memory collectives unavailable", "comm_path": comm_path,
                              "health": comm.health, "fused_error": getattr(comm, "fused_error", None)}))
        return 3
    max_len = ((S + 2 * (K + W) + 80 + 15) // 16) * 16
    eng = LlmEngine(model, EngineConfig(max_batch=B, max_seq_len=max_len, prefill_token_budget=8192))
    runner = eng.runner
    g = torch.Generator().manual_seed(1234)
    prompts = [torch.randint(0, cfg.vocab_size, (S,), generator=g).tolist() for _ in range(B)]

    def sync_all():
        comm.barrier()
        torch.cuda.synchronize()

    def timed_multi(run, seqs, toks, steps):
        """One timed region of exactly `steps` decode steps: barrier + synchronize on both sides, CUDA events, max
        over ranks. The sequences are rolled back afterwards so that every region decodes the same positions."""
        base = [s.length for s in seqs]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record()
        out = run.decode_multi(seqs, toks, steps)
        e1.record()
        sync_all()
        ms = comm.max_over_ranks(e0.elapsed_time(e1))
        for s, n in zip(seqs, base):
            s.truncate(n)
        return ms, out

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
            ms = statistics.median(timed_multi(runner, seqs, toks, n)[0] for _ in range(3))
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
    region_ms = []
    for _ in range(R):                                # R regions of EXACTLY K timed steps each; the median is reported
        ms, out = timed_multi(runner, seqs, toks, K)
        region_ms.append(ms)
    launches = runner.launches_last
    ms_total = statistics.median(region_ms)
    ms_step = ms_total / K
    value = B * K / ms_total * 1e3
    extra.update(repeats=R, value_min=round(B * K / max(region_ms) * 1e3, 1),
                 value_max=round(B * K / min(region_ms) * 1e3, 1))

    # ---- end to end through the per-step public API --------------------------------------------------
    e2e_regions = []
    for rep in range(3):
        base = [s.length for s in seqs]
        tk = toks
        for _ in range(W if rep == 0 else 1):
            tk = runner.decode(seqs, tk).tolist()
        sync_all()
        t0 = time.perf_counter()
        for _ in range(K):
            tk = runner.decode(seqs, tk).tolist()     # H2D metadata + graph + D2H tokens + sync, every step
        torch.cuda.synchronize()
        comm.barrier()
        e2e_regions.append(comm.max_over_ranks(time.perf_counter() - t0))
        for s, n in zip(seqs, base):
            s.truncate(n)
    e2e_s = statistics.median(e2e_regions)
    h2d, d2h = runner.h2d_bytes_last, runner.d2h_bytes_last
    clocks = sampler.stop() if comm.rank == 0 else {}

    # ---- same process, same N: the library-collective arm (NCCL all-reduce + separate norm kernels) -----
    vs_baseline = None
    if world > 1 and comm_path == "fused" and not args.no_baseline:
        import copy
        import dataclasses

        base_model = copy.copy(model)
        base_model.comm = dataclasses.replace(comm, fused=None)
        base_model._chain_ok = False
        base_runner = type(runner)(base_model, eng.pool, max_batch=B, max_seq_len=max_len)
        ob = base_runner.decode_multi(seqs, toks, W)
        for s in seqs:
            s.truncate(s.length - W)
        ms_b = statistics.median(timed_multi(base_runner, seqs, toks, K)[0] for _ in range(3))
        extra["nccl_unfused_tok_s"] = round(B * K / ms_b * 1e3, 1)
        extra["nccl_unfused_ms_per_step"] = round(ms_b / K, 4)
        vs_baseline = round(value / (B * K / ms_b * 1e3), 3)
        del base_runner, base_model, ob

    # ---- TP = N produces the tokens of TP = 1 on the same weights (teacher forced, checked on rank 0) --
    if world > 1 and not invalid:
        extra.update(tp_equivalence(model, comm, cfg, dev))

    st = None
    try:
        from inference_b200 import ops

        st = ops.device_status()
    except Exception:
        pass
    health = comm.health
    for s in seqs:
        s.release()
    del runner, eng, model, seqs
    torch.cuda.empty_cache()

    if not args.no_dit and not invalid:
        try:
            extra.update(dit_section(comm, dev))
        except Exception as e:  # noqa: BLE001
            extra["dit_error"] = f"{type(e).__name__}: {str(e)[:300]}"

    if comm.rank == 0:
        line = {
            "metric": "llama3_8b_decode_tokens_per_s", "value": round(value, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": vs_baseline, "dtype": "bf16",
            "data": "synthetic: uniform-random prompt ids, random-init N(0,0.02) weights",
            "config": {"model": "Llama-3-8B (32L, h4096, 32/8 heads, ffn 14336, vocab 128256)", "global_batch": B,
                       "seq_len": S, "decode_steps": K, "parallelism": f"tp{world}", "kv_block": 16,
                       "l2_policy": "inputs larger than L2 (16 GB of weights + KV streamed every step)",
                       "sampling": "greedy on device",
                       "vs_baseline_is": "value / this repo's NCCL all-reduce + unfused-norm arm at the same N, same "
                                         "process (the reference publishes no number for this configuration)"},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                       "reasons": clocks.get("reasons", []), "samples": clocks.get("samples", 0)},
            "e2e": {"value": round(B * K / e2e_s, 1), "unit": "tokens/s", "ms_per_step": round(e2e_s / K * 1e3, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "impl": "ours", "comm_path": comm_path, "health": health,
            "fused_error": getattr(comm, "fused_error", None), "extra": extra,
        }
        if st is not None:
            line["device_status"] = st[0]
        if invalid:
            line["invalid"] = invalid
        print(json.dumps(line))
    comm.barrier()
    return 0


def tp_equivalence(model, comm, cfg, dev) -> dict:
    """All ranks: 4 prompts of 48 tokens, first token + 8 teacher-forced decode steps at TP = N; rank 0 repeats them on
    the gathered TP = 1 model. A position matches when the tokens agree, or when the TP = 1 logit margin between the two
    candidates is inside the measured logit error (a tie that bf16 partial sums may break either way)."""
    import torch

    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner

    g = torch.Generator().manual_seed(99)
    prompts = [torch.randint(0, cfg.vocab_size, (48,), generator=g).tolist() for _ in range(4)]
    full = model.gather_unsharded(0)

    def run(m, forced=None):
        pool = PagedKvPool(cfg.num_layers, 4 * 8, m.hkv, cfg.head_dim, 16, device=dev)
        r = ModelRunner(m, pool, max_batch=4, max_seq_len=128, use_graphs=False)
        seqs = [PagedSequence(pool) for _ in prompts]
        lg = [r.prefill(seqs, prompts, want_logits=True).float().cpu()]
        for k in range(8):
            feed = forced[k] if forced is not None else lg[-1].argmax(-1).tolist()
            lg.append(r.decode(seqs, feed, want_logits=True).float().cpu())
        for s in seqs:
            s.release()
        return lg

    ok, err, tok_equal = True, 0.0, True
    forced_t = torch.zeros((8, 4), dtype=torch.int64, device=dev)
    ref = None
    if comm.rank == 0:
        ref = run(full)
        forced_t.copy_(torch.stack([l.argmax(-1) for l in ref[:8]]))
    comm.broadcast(forced_t, 0)
    got = run(model, forced_t.tolist())
    if comm.rank == 0:
        for a, b in zip(ref, got):
            e = (a - b).abs().max().item()
            err = max(err, e)
            ta, tb = a.argmax(-1), b.argmax(-1)
            for i in range(a.shape[0]):
                if ta[i] != tb[i]:
                    tok_equal = False
                    if (a[i, ta[i]] - a[i, tb[i]]).item() > 2 * e:
                        ok = False
    del full
    torch.cuda.empty_cache()
    return {"tp_matches_tp1": bool(ok), "tp_tokens_identical": bool(tok_equal), "tp_vs_tp1_max_logit_err": round(err, 5)}


if __name__ == "__main__":
    rc = main()
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    sys.exit(rc)
