"""Worker for the multi-GPU tensor-parallel tests (launched by torch.distributed.run, one rank per GPU)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from inference_b200 import ops
    from inference_b200.engine.kv_pool import PagedKvPool, PagedSequence
    from inference_b200.engine.runner import ModelRunner
    from inference_b200.models import ModelConfig
    from inference_b200.models.llama import LlamaGpu
    from inference_b200.models.oracle import OracleLlama, random_llama_weights
    from inference_b200.parallel import init_distributed
    from inference_b200.parallel.symm import FusedCollectives

    mode = sys.argv[1] if len(sys.argv) > 1 else "fused"
    comm = init_distributed()
    dev = comm.device
    P, r = comm.world, comm.rank

    # 1. fused all-reduce + residual + rmsnorm against a torch reference
    H = 1024
    fc = FusedCollectives(comm, H, max_tokens=64)
    g = torch.Generator(device=dev).manual_seed(100 + r)
    for T in (1, 7, 64):
        for it in range(3):
            part = (torch.randn(T, H, device=dev, generator=g) * 0.5).bfloat16()
            allp = comm.all_gather(part[None], dim=0).float()           # [P, T, H]
            res = (torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + it)) * 0.5) \
                .bfloat16()
            w = (torch.rand(H, device=dev, generator=torch.Generator(device=dev).manual_seed(9)) + 0.5).bfloat16()
            buf, i = fc.exchange_buffer(T)
            buf.copy_(part)
            res_k = res.clone()
            out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
            fc._launch(i, T, res_k, w, 1e-5, 0.0, out)
            torch.cuda.synchronize()
            s = (allp.sum(0) + res.float()).bfloat16()
            assert torch.equal(res_k, s), f"rank {r}: residual mismatch T={T}"
            sf = s.float()
            ref = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
            assert (out.float() - ref).abs().max().item() < 3e-2, f"rank {r}: norm mismatch T={T}"
            t2 = part.clone()
            fc.all_reduce(t2)
            torch.cuda.synchronize()
            assert (t2.float() - allp.sum(0)).abs().max().item() < 2e-2
    fc.check()

    # 1b. row-parallel decode GEMM with the cross-rank sum in its epilogue (one-shot and two-shot), against torch;
    #     every rank must hold bit-identical rows, and the sums of squares must describe exactly what was stored
    for mode_id in (1, 2):
        fc.reduce_mode = mode_id
        for T, Kl in ((1, 512), (7, 256), (64, 1792 // 7 * 2)):
            for it in range(3):
                gk = torch.Generator(device=dev).manual_seed(1000 * mode_id + 10 * T + it + 100 * r)
                a = (torch.randn(T, Kl, device=dev, generator=gk) * 0.5).bfloat16()
                wgt = (torch.randn(H, Kl, device=dev, generator=gk) * 0.05).bfloat16()
                res0 = (torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(it)) * 0.5) \
                    .bfloat16()
                part = (a.float() @ wgt.float().t()).bfloat16()
                allp = comm.all_gather(part[None], dim=0).float()
                want = (allp.sum(0) + res0.float()).bfloat16()
                res = res0.clone()
                ssq, other = ops.ssq_buffer(dev), ops.ssq_buffer(dev).fill_(5)
                fc.gemm_peer_reduce(a, wgt, res, it & 1, ssq_out=ssq, ssq_zero=other)
                torch.cuda.synchronize()
                fc.check()
                err = (res.float() - want.float()).abs().max().item()
                assert err < 0.06, f"rank {r}: peer-reduce GEMM mode {mode_id} T={T} err {err}"
                allr = comm.all_gather(res.clone()[None], dim=0)
                assert all(torch.equal(allr[0], allr[k]) for k in range(P)), f"mode {mode_id}: ranks differ"
                got_ss = ops.ssq_values(ssq)[:T]
                ref_ss = res.float().pow(2).sum(-1)
                assert torch.allclose(got_ss, ref_ss, rtol=1e-4, atol=1e-4), f"mode {mode_id} T={T}: ssq"
                assert int(other.abs().sum()) == 0, "the other accumulator was not cleared"
                allq = comm.all_gather(ssq[None], dim=0)
                assert all(torch.equal(allq[0], allq[k]) for k in range(P)), "sums of squares differ between ranks"
                comm.barrier()
    fc.reduce_mode = 0

    # 2. TP=k model == TP=1 oracle within bf16 tolerance, through prefill and graph decode
    cfg = ModelConfig.from_json({"hidden_size": 1024, "intermediate_size": 2048, "num_hidden_layers": 2,
                                 "num_attention_heads": 8, "num_key_value_heads": 8, "head_dim": 128,
                                 "vocab_size": 4096, "rope_theta": 10000.0})
    w = {k: v.bfloat16().float() for k, v in random_llama_weights(cfg, seed=1, std=0.05).items()}
    oracle = OracleLlama(cfg, w, dtype=torch.float32, device=dev)
    if mode == "fused":
        from inference_b200.parallel.symm import attach_fused

        attach_fused(comm)
    model = LlamaGpu(cfg, comm=comm, device=dev).load_state_dict(w)
    assert (comm.fused is not None) == (mode == "fused")
    assert model.norm_folded == (mode == "fused") and model._chain_ok == (mode == "fused")
    pool = PagedKvPool(cfg.num_layers, 64, model.hkv, cfg.head_dim, 16, device=dev)
    runner = ModelRunner(model, pool, max_batch=4, max_seq_len=256)
    prompts = [list(range(3, 40)), list(range(100, 109))]
    seqs = [PagedSequence(pool) for _ in prompts]
    logits = runner.prefill(seqs, prompts, want_logits=True)
    caches = []
    for i, p in enumerate(prompts):
        c = oracle.make_cache()
        ref = oracle.decode_logits(torch.tensor([p], device=dev), c, 0)[0]
        caches.append(c)
        assert (logits[i] - ref).abs().max().item() < 0.08 * max(1.0, ref.abs().max().item()), f"prefill seq {i}"
    toks = [int(logits[i].argmax()) for i in range(2)]
    for step in range(4):
        lg = runner.decode(seqs, toks, want_logits=True)
        for i in range(2):
            ref = oracle.decode_logits(torch.tensor([[toks[i]]], device=dev), caches[i], caches[i].offset)[0]
            assert (lg[i] - ref).abs().max().item() < 0.08 * max(1.0, ref.abs().max().item()), f"decode {step} {i}"
        toks = [int(lg[i].argmax()) for i in range(2)]
    got = runner.decode(seqs, toks).tolist()
    allg = comm.all_gather(torch.tensor([got], device=dev), dim=0)
    assert all(torch.equal(allg[0], allg[k]) for k in range(P)), "ranks disagree on sampled tokens"
    # vocabulary-parallel greedy head (fused: candidates exchanged through peer memory) equals argmax of all logits
    gh = torch.Generator(device=dev).manual_seed(123)
    for rows in (1, 7, 64):
        hid = torch.randn(rows, cfg.hidden_size, device=dev, generator=gh).bfloat16()
        want = model.logits(hid).argmax(-1)
        got_ids = model.greedy_tokens(hid)
        assert torch.equal(want, got_ids), f"distributed argmax rows={rows}"
    for s_ in seqs:
        s_.release()
    # 3. prompts longer than the decode-sized exchange buffers: fused reduce-scatter / all-gather prefill path
    #    (odd total length so the row shards are uneven) against the oracle
    pool2 = PagedKvPool(cfg.num_layers, 128, model.hkv, cfg.head_dim, 16, device=dev)
    runner2 = ModelRunner(model, pool2, max_batch=4, max_seq_len=1024)
    long_prompts = [[(7 * i + 3) % cfg.vocab_size for i in range(301)], [(5 * i + 11) % cfg.vocab_size for i in range(170)]]
    seqs2 = [PagedSequence(pool2) for _ in long_prompts]
    if mode == "fused":
        assert model._use_tp_prefill(sum(len(p) for p in long_prompts))
    for rep in range(2):
        lg2 = runner2.prefill(seqs2, long_prompts, want_logits=True)
        for i, p in enumerate(long_prompts):
            ref = oracle.decode_logits(torch.tensor([p], device=dev), oracle.make_cache(), 0)[0]
            err = (lg2[i] - ref).abs().max().item()
            assert err < 0.1 * max(1.0, ref.abs().max().item()), f"long prefill seq {i} rep {rep} err {err}"
        for s_ in seqs2:
            s_.release()
        seqs2 = [PagedSequence(pool2) for _ in long_prompts]
    ops.check_status()
    comm.barrier()
    if r == 0:
        print(f"TP_WORKER_OK world={P} mode={mode}")


if __name__ == "__main__":
    main()
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
