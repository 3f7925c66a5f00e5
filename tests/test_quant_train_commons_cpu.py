"""Adapters (LoRA / LoKr / LoHa), trainer optimisers and gradient helpers, 8-bit linears, ConvRot, MLX repack."""
import numpy as np
import pytest
import torch


def test_lokr_residual_equals_dense_delta_and_adaptlinear_merge():
    from inference_b200.media.adapters import AdaptLinear, LokrFactors, reconstruct_lokr_delta

    g = torch.Generator().manual_seed(0)
    out_f, in_f = 12, 20                       # a*b = 12 (3*4), c*d = 20 (4*5)
    w = torch.randn(out_f, in_f, generator=g)
    w1, w2 = torch.randn(3, 4, generator=g), torch.randn(4, 5, generator=g)
    alpha, rank = 4.0, 8.0
    f = LokrFactors.build(alpha / rank, (out_f, in_f), w1=w1, w2=w2)
    x = torch.randn(2, 7, in_f, generator=g)
    delta = reconstruct_lokr_delta(w1=w1, w2=w2, alpha=alpha, rank=rank, scale=1.0, base_shape=(out_f, in_f))
    torch.testing.assert_close(f.residual(x), x @ delta.t(), atol=1e-5, rtol=1e-5)
    # low-rank legs, and shapes that cannot be applied structurally
    a, b = torch.randn(4, 2, generator=g), torch.randn(2, 5, generator=g)
    f2 = LokrFactors.build(1.0, (out_f, in_f), w1=w1, w2_a=a, w2_b=b)
    torch.testing.assert_close(f2.residual(x), x @ torch.kron(w1, a @ b).t(), atol=1e-5, rtol=1e-5)
    assert LokrFactors.build(1.0, (out_f, in_f + 1), w1=w1, w2=w2) is None
    assert LokrFactors.build(1.0, (out_f, in_f), w1=w1, w2=w2, w2_t2=torch.zeros(1)) is None
    with pytest.raises(ValueError, match="w1 missing"):
        LokrFactors.build(1.0, (out_f, in_f), w2=w2)
    lin = AdaptLinear.from_dense(w, torch.randn(out_f, generator=g))
    assert not lin.is_adapted() and not lin.is_packed()
    la, lb = torch.randn(3, in_f, generator=g), torch.randn(out_f, 3, generator=g)
    lin.push_lora(la, lb, 0.5)
    lin.push_lokr_structured(f)
    ref = x @ (w + 0.5 * lb @ la + delta).t() + lin.bias
    torch.testing.assert_close(lin(x), ref, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(lin.merged_weight(), w + 0.5 * lb @ la + delta, atol=1e-5, rtol=1e-5)
    lin.clear_adapters()
    torch.testing.assert_close(lin(x), x @ w.t() + lin.bias)
    packed = AdaptLinear.from_packed(lambda t: t @ w.t(), in_f, out_f)
    packed.push_lora(la, lb, 1.0)
    torch.testing.assert_close(packed(x), x @ (w + lb @ la).t(), atol=1e-4, rtol=1e-4)


def test_thirdparty_lokr_loha_deltas():
    from inference_b200.media.adapters import ThirdPartyLoha, parse_thirdparty, reconstruct_loha_delta

    t = torch.tensor
    d = reconstruct_loha_delta(t([[1.0], [2.0]]), t([[3.0, 4.0]]), t([[1.0], [0.0]]), t([[5.0, 6.0]]), 0.5, (2, 2))
    assert d.flatten().tolist() == [7.5, 12.0, 0.0, 0.0]
    files = {"m.lokr_w1": torch.eye(2), "m.lokr_w2_a": torch.ones(2, 4), "m.lokr_w2_b": torch.ones(4, 3),
             "m.alpha": t(2.0), "n.hada_w1_a": torch.ones(2, 2), "n.hada_w1_b": torch.ones(2, 2),
             "n.hada_w2_a": torch.ones(2, 2), "n.hada_w2_b": torch.ones(2, 2)}
    lokr, loha = parse_thirdparty(files)
    assert set(lokr) == {"m"} and set(loha) == {"n"}
    assert lokr["m"].rank() == 4.0 and lokr["m"].lycoris_scale() == 0.5
    torch.testing.assert_close(lokr["m"].delta((4, 6), 2.0), torch.kron(torch.eye(2), torch.full((2, 3), 4.0)))
    assert loha["n"].lycoris_scale() == 1.0 and float(loha["n"].delta((2, 2), 1.0)[0, 0]) == 4.0
    with pytest.raises(ValueError, match="factor is missing"):
        ThirdPartyLoha(w1_a=torch.ones(1, 1)).delta((1, 1), 1.0)


def test_optimizer_names_and_gradient_helpers():
    from inference_b200.media import train_optim as o

    for alias, want in [("adamw", "adamw"), ("AdamW", "adamw"), ("adamw8bit", "adamw"), ("AdamW-8bit", "adamw"),
                        ("adamw_8bit", "adamw"), ("adam8bit", "adamw"), ("adam", "adam"), ("prodigy-opt", "prodigy"),
                        ("rose_opt", "rose")]:
        assert o.normalize(alias) == want
    assert o.normalize("adamax") == "adamax" and not o.is_supported("adamax") and not o.is_supported("lion")
    with pytest.raises(ValueError, match="unsupported optimizer"):
        o.TrainOptimizer("radam", [], 1e-3, 0.0)
    p, q = torch.zeros(2, 2), torch.zeros(3)
    grads = {id(p): torch.full((2, 2), 3.0), id(q): torch.full((3,), 4.0)}
    norm = o.clip_grad_norm(grads, [p, q], 1.0)
    assert abs(norm - (4 * 9 + 3 * 16) ** 0.5) < 1e-9
    after = sum(float(g.pow(2).sum()) for g in grads.values()) ** 0.5
    assert abs(after - 1.0) < 1e-5
    acc = o.accumulate_grads(None, {id(p): torch.ones(2, 2)}, [p, q])
    acc = o.accumulate_grads(acc, {id(p): torch.ones(2, 2), id(q): torch.ones(3)}, [p, q])
    assert float(acc[id(p)][0, 0]) == 2.0 and float(acc[id(q)][0]) == 1.0
    o.scale_grads(acc, [p, q], 0.5)
    assert float(acc[id(p)][0, 0]) == 1.0
    assert o.file_stem("my_style.safetensors") == "my_style" and o.file_stem("noext") == "noext"
    assert o.checkpoint_filename("my_style", 500) == "my_style-step000500.safetensors"
    assert o.checkpoint_filename("s", 90) < o.checkpoint_filename("s", 100)
    assert [o.bucket_resolution(r) for r in (0, 20, 512, 1000, 1024)] == [512, 32, 512, 992, 1024]


# Rose centres each row's gradient, so the row-mean component of the error is never corrected: it plateaus higher
@pytest.mark.parametrize("name,lr,steps,frac", [("adamw", 0.05, 200, 0.05), ("rose", 0.02, 300, 0.3),
                                                ("prodigy", 1.0, 300, 0.05)])
def test_optimizers_minimise_a_least_squares_problem(name, lr, steps, frac):
    from inference_b200.media import train_optim as o

    g = torch.Generator().manual_seed(3)
    a_true, x = torch.randn(6, 4, generator=g), torch.randn(64, 4, generator=g)
    y = x @ a_true.t()
    a = (torch.randn(6, 4, generator=g) * 0.1).requires_grad_(True)
    opt = o.TrainOptimizer(name, [a], lr, 0.0)
    first = None
    for i in range(steps):
        loss = ((x @ a.t() - y) ** 2).mean()
        first = first if first is not None else float(loss.detach())
        opt.set_lr_scaled(1.0 - i / steps)              # linear decay, as the trainers' schedules do
        opt.step(o.grads_of(loss, [a]))
    assert float(((x @ a.t() - y) ** 2).mean().detach()) < frac * first


def test_rose_update_rules_and_prodigy_defaults():
    from inference_b200.media.train_optim import Prodigy, Rose

    r = Rose([], 0.1, 0.0)
    g = torch.tensor([[1.0, -1.0, 3.0], [0.0, 0.0, 0.0]])
    new = r.update_one(torch.zeros(2, 3), g)
    assert torch.all(new[1] == 0)                       # a zero-gradient row divides by 1, not by 0
    assert new[0, 2] < 0 < new[0, 1]
    v = r.update_one(torch.zeros(3), torch.tensor([2.0, -2.0, 0.0]))
    torch.testing.assert_close(v, torch.tensor([-0.05, 0.05, 0.0]))
    with pytest.raises(ValueError):
        r.update_one(torch.tensor(0.0), torch.tensor(1.0))
    assert Prodigy([], 1e-4, 0.0).lr == 1.0 and Prodigy([], 0.5, 0.0).lr == 0.5


def test_checkpointed_backward_matches_plain_autograd():
    from inference_b200.media.train_optim import checkpointed_backward, grads_of

    g = torch.Generator().manual_seed(5)
    ws = [torch.randn(8, 8, generator=g).mul_(0.3).requires_grad_(True) for _ in range(4)]
    segs = [(lambda h, w=w: torch.tanh(h @ w)) for w in ws]
    x = torch.randn(5, 8, generator=g)
    loss_fn = lambda out: (out ** 2).sum()
    h = x
    for s in segs:
        h = s(h)
    ref = grads_of(loss_fn(h), ws)
    loss, got = checkpointed_backward(segs, x, loss_fn, ws)
    assert abs(loss - float(loss_fn(h))) < 1e-5
    for w in ws:
        torch.testing.assert_close(got[id(w)], ref[id(w)], atol=1e-5, rtol=1e-5)


def test_eight_bit_linears_and_convrot():
    from inference_b200.ops import eight_bit as e

    g = torch.Generator().manual_seed(7)
    w, b, x = torch.randn(24, 64, generator=g) * 0.1, torch.randn(24, generator=g), torch.randn(2, 5, 64, generator=g)
    ref = x @ w.t() + b
    for layer, tol in ((e.Fp8Linear(w, b), 0.08), (e.Int8Linear(w, b), 0.03), (e.Int8Linear(w, b, per_channel=True), 0.03)):
        y = layer(x)
        assert y.shape == ref.shape and float((y - ref).norm() / ref.norm()) < tol
    q, s = e.quantize_int8(torch.tensor([[1.0, -2.0, 0.5]]))
    assert q.tolist() == [[64, -127, 32]] and abs(s - 2 / 127) < 1e-9
    q, s = e.quantize_fp8(torch.zeros(2, 2))
    assert s > 0 and float(q.float().abs().max()) == 0
    wq, sc = e.quantize_int8_per_channel(w)
    again = e.Int8Linear.from_per_channel_parts(wq, sc, b)
    torch.testing.assert_close(again(x), e.Int8Linear(w, b, per_channel=True)(x))
    with pytest.raises(ValueError):
        e.Int8Linear.from_per_channel_parts(wq, sc[:-1])
    assert all(e.is_power_of_four(n) for n in (1, 4, 16, 64, 256, 1024, 4096))
    assert not any(e.is_power_of_four(n) for n in (0, 2, 8, 32, 128, 512, 3, 6))
    for n in (4, 16, 64, 256):
        r = e.regular_hadamard(n)
        assert float((r @ r.t() - torch.eye(n)).abs().max()) < 1e-5 and float((r - r.t()).abs().max()) < 1e-6
        assert float((r.sum(1) - r.sum(1)[0]).abs().max()) < 1e-5          # regular: constant row sums
    assert e.regular_hadamard(4).tolist()[0] == [0.5, 0.5, 0.5, -0.5]
    with pytest.raises(ValueError):
        e.regular_hadamard(8)
    r = e.regular_hadamard(16)
    xr, wr = e.convrot_rotate(x, r), e.convrot_rotate(w, r)
    torch.testing.assert_close(xr @ wr.t(), x @ w.t(), atol=1e-4, rtol=1e-4)
    spike = torch.zeros(1, 16)
    spike[0, 3] = 16.0
    assert float(e.convrot_rotate(spike, r).abs().max()) == 4.0          # the outlier is spread over its group
    with pytest.raises(ValueError):
        e.convrot_rotate(torch.zeros(1, 10), r)


@pytest.mark.parametrize("group", [64, 32])
def test_mlx_repack_is_lossless(group):
    from inference_b200.io import mlx_repack as m
    from inference_b200.io.gguf_quants import dequantize

    g = torch.Generator().manual_seed(11)
    w = torch.randn(6, 256, generator=g)
    wq, sc, bi = m.pack_mlx_affine(w, 4, group)
    sc, bi = sc.half().float(), bi.half().float()       # a checkpoint stores fp16 scales / biases
    assert wq.shape == (6, 32) and m.mlx_packed_bits(wq.shape[1], sc.shape[1], group) == 4
    ref = m.dequant_mlx_q4_reference(wq, sc, bi, group)
    assert float((ref - w).abs().max()) < float((w.max() - w.min())) / 15
    q41 = m.repack_mlx_q4_to_q4_1(wq, sc, bi, group)
    assert q41.shape == (6, 256 // 32 * 20)
    got = torch.from_numpy(dequantize(q41.numpy().reshape(-1), "Q4_1", 6 * 256).copy()).reshape(6, 256)
    assert torch.equal(got, ref)
    wq8, sc8, bi8 = m.pack_mlx_affine(w, 8, group)
    assert m.mlx_packed_bits(wq8.shape[1], sc8.shape[1], group) == 8
    assert float((m.dequant_mlx_q8(wq8, sc8, bi8, group) - w).abs().max()) < float(w.max() - w.min()) / 255
    assert m.f16_exact(0.5) and not m.f16_exact(0.1)
    with pytest.raises(ValueError, match="not an MLX"):
        m.dequant_mlx_q4_reference(wq, sc[:, :-1], bi[:, :-1], group)
    with pytest.raises(ValueError):
        m.pack_mlx_affine(w, 3, group)
