"""FLUX-shaped DiT benchmark: ms per denoise step and seconds per 1024x1024 image (28 Euler flow-matching steps
plus the VAE decode when --vae is given) on random weights and synthetic conditioning, device-timed with CUDA events."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=28)
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--depth", type=int, default=19)
    ap.add_argument("--depth-single", type=int, default=38)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--eager", action="store_true", help="launch every kernel from Python instead of replaying a graph")
    ap.add_argument("--vae", action="store_true", help="also time the VAE decode of the final latents")
    args = ap.parse_args()
    from inference_b200.contracts.gen_core.sampling import build_flow_sigmas, compute_mu, image_seq_len
    from inference_b200 import ops
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, make_ids, rope_table

    from inference_b200.parallel import init_distributed

    comm = init_distributed()          # world 1 unless launched by torch.distributed.run (then sequence parallel)
    dev = comm.device
    cfg = FluxConfig(depth=args.depth, depth_single=args.depth_single)
    model = FluxDiTGpu(cfg, comm=comm, device=dev).init_random(0)
    ht = args.size // 16
    Si, St = ht * ht, 512
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(1, Si, 64, device=dev, generator=g).bfloat16()
    txt = torch.randn(1, St, 4096, device=dev, generator=g).bfloat16()
    y = torch.randn(1, 768, device=dev, generator=g).bfloat16()
    txt_ids, img_ids = make_ids(ht, ht, St, dev)
    rope = rope_table(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.theta)
    gd = torch.full((1,), 3.5, device=dev)
    sigmas = build_flow_sigmas(args.steps, compute_mu(image_seq_len(args.size, args.size), args.steps))

    def run(n_steps):
        lat = x
        for i in range(n_steps):
            t = torch.full((1,), sigmas[i], device=dev)
            fwd = model.forward if args.eager else model.forward_graphed
            v = fwd(lat, img_ids, txt, txt_ids, t, y, gd, rope=rope)
            lat = ops.axpy(1.0, lat, sigmas[i + 1] - sigmas[i], v.contiguous())
        return lat

    run(args.warmup)
    comm.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run(args.steps)
    e1.record()
    torch.cuda.synchronize()
    ms = comm.max_over_ranks(e0.elapsed_time(e1))
    S = Si + St
    H, M = cfg.hidden_size, cfg.mlp_hidden
    flops_double = 2 * S * H * (3 * H + H + 2 * M) + 4 * S * S * H
    flops_single = 2 * S * H * (3 * H + M) + 2 * S * (H + M) * H + 4 * S * S * H
    tflop = (cfg.depth * flops_double + cfg.depth_single * flops_single) / 1e12
    vae_ms = None
    if args.vae and comm.rank == 0:
        from inference_b200.models.vae import VaeConfig, VaeDecoderGpu

        vae = VaeDecoderGpu(VaeConfig(), dev).init_random(1)
        z = torch.randn(1, 16, args.size // 8, args.size // 8, device=dev, generator=g)
        vae.decode_rgb8(z)
        torch.cuda.synchronize()
        e0.record()
        img = vae.decode_rgb8(z)
        e1.record()
        torch.cuda.synchronize()
        vae_ms = round(e0.elapsed_time(e1), 2)
        assert img.shape == (1, args.size, args.size, 3)
    ops.check_status()
    comm.barrier()
    phases = None
    if os.environ.get("SWB_SP_TRACE") == "1" and comm.world > 1:
        t = torch.full((1,), 0.5, device=dev)
        model.forward(x, img_ids, txt, txt_ids, t, y, gd, rope=rope)     # eager, with phase events
        phases = getattr(model, "sp_phase_ms", None)
    comm.barrier()
    if comm.rank != 0:
        return
    import os as _os
    print(json.dumps({"n_gpus": comm.world, "sp_impl": _os.environ.get("SWB_SP", "fused") if comm.world > 1 else None,
                      "metric": "flux_dit_ms_per_step", "cuda_graph": not args.eager, "sp_phase_ms": phases, "ms_per_step": round(ms / args.steps, 3),
                      "s_per_image_dit_only": round(ms / 1e3, 3), "steps": args.steps, "size": args.size,
                      "tflop_per_step": round(tflop, 2), "achieved_tflops": round(tflop / (ms / args.steps) * 1e3, 1),
                      "launches_per_step": model.launches, "weights_gb": round(model.weight_bytes() / 1e9, 2), "vae_decode_ms": vae_ms,
                      "s_per_image": round((ms + (vae_ms or 0.0)) / 1e3, 3)}))


if __name__ == "__main__":
    main()
