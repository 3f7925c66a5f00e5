"""Worker for the sequence-parallel DiT tests (torch.distributed.run, one rank per GPU): the SP forward (fused peer
stores, or the NCCL all-to-all baseline with SWB_SP=nccl) must match the single-GPU forward of the same weights."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from inference_b200 import ops
    from inference_b200.models.dit_flux import FluxConfig, FluxDiTGpu, make_ids, random_flux_weights, rope_table
    from inference_b200.parallel import init_distributed

    comm = init_distributed()
    dev, P, r = comm.device, comm.world, comm.rank
    cfg = FluxConfig(in_channels=64, vec_in_dim=32, context_in_dim=64, hidden_size=1024, num_heads=8, depth=2,
                     depth_single=2)
    w = random_flux_weights(cfg, seed=3, std=0.03)
    single = FluxDiTGpu(cfg, device=dev).load_state_dict(w)
    par = FluxDiTGpu(cfg, comm=comm, device=dev).load_state_dict(w)
    ht, wt, St = 16, 24, 128
    g = torch.Generator(device=dev).manual_seed(11)
    img = torch.randn(1, ht * wt, 64, device=dev, generator=g).bfloat16()
    txt = torch.randn(1, St, 64, device=dev, generator=g).bfloat16()
    y = torch.randn(1, 32, device=dev, generator=g).bfloat16()
    txt_ids, img_ids = make_ids(ht, wt, St, dev)
    rope = rope_table(torch.cat([txt_ids, img_ids], 0), cfg.axes_dim, cfg.theta)
    t = torch.full((1,), 0.6, device=dev)
    gd = torch.full((1,), 3.5, device=dev)
    ref = single.forward(img, img_ids, txt, txt_ids, t, y, gd, rope=rope).float()
    for it in range(3):                       # repeated calls reuse the symmetric buffers and flag epochs
        out = par.forward(img, img_ids, txt, txt_ids, t, y, gd, rope=rope).float()
        torch.cuda.synchronize()
        ops.check_status()
        err = (out - ref).abs().max().item()
        tol = 0.05 * max(1.0, ref.abs().max().item())
        assert out.shape == ref.shape and err < tol, (it, err, tol)
    for it in range(2):                       # graph capture + replay of the sequence-parallel forward
        out = par.forward_graphed(img, img_ids, txt, txt_ids, t, y, gd, rope=rope).float()
        torch.cuda.synchronize()
        ops.check_status()
        assert (out - ref).abs().max().item() < tol, ("graph", it)
    comm.barrier()
    if r == 0:
        print(f"SP_WORKER_OK world={P} mode={os.environ.get('SWB_SP', 'fused')} err={err:.4f}")


if __name__ == "__main__":
    main()
