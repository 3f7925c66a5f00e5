"""Device temperature / top-k / top-p sampler: exact cases (top_k = 1, tiny top_p, masks, the kept-set boundary with
ties) and the empirical distribution of many draws against the analytic one."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _probs(logits, temperature, top_k, top_p, allow=None):
    """fp64 reference of the kept, renormalised distribution (ties at the boundary admitted in index order)."""
    l = logits.double().clone()
    if allow is not None:
        l[allow == 0] = float("-inf")
    w = torch.exp((l - l.max()) / temperature)
    order = sorted(range(len(w)), key=lambda i: (-w[i].item(), i))
    keep, mass, z = [], 0.0, w.sum().item()
    for i in order:
        if w[i] <= 0:
            break
        if top_k > 0 and len(keep) >= top_k:
            break
        if top_p < 1.0 and mass >= top_p * z:
            break
        keep.append(i)
        mass += w[i].item()
    p = torch.zeros_like(w)
    p[keep] = w[keep] / mass
    return p


def test_exact_cases():
    from inference_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(0)
    logits = torch.randn(6, 50000, device="cuda", generator=g)
    u = torch.rand(6, device="cuda", generator=g)
    am = logits.argmax(-1)
    assert torch.equal(ops.sample_device(logits, 0.8, 1, 1.0, u), am)                    # top_k = 1
    assert torch.equal(ops.sample_device(logits, 0.8, 0, 1e-6, u), am)                   # nucleus of one token
    assert torch.equal(ops.sample_device(logits.bfloat16(), 1.3, 1, 1.0, u), logits.bfloat16().float().argmax(-1))
    allow = torch.zeros(50000, dtype=torch.uint8, device="cuda")
    allow[[7, 4242, 31000]] = 1
    for _ in range(5):
        t = ops.sample_device(logits, 2.0, 0, 1.0, torch.rand(6, device="cuda", generator=g), allow_mask=allow)
        assert set(t.tolist()) <= {7, 4242, 31000}
    none = torch.full((2, 100), float("-inf"), device="cuda")
    assert ops.sample_device(none, 1.0, 0, 1.0, u[:2]).tolist() == [0, 0]
    # u sweeps the CDF in index order over the kept set: four equal logits, top_k = 2 keeps the first two of the tie
    tie = torch.full((1, 1000), -10.0, device="cuda")
    tie[0, [100, 200, 300, 400]] = 5.0
    picks = {int(ops.sample_device(tie, 1.0, 2, 1.0, torch.tensor([x], device="cuda"))) for x in (0.0, 0.3, 0.6, 0.99)}
    assert picks == {100, 200}
    prob = torch.empty(1, device="cuda")
    ops.sample_device(tie, 1.0, 2, 1.0, torch.tensor([0.1], device="cuda"), out_prob=prob)
    assert abs(prob.item() - 0.5) < 1e-6
    ops.check_status()


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 40, 1.0), (1.2, 0, 0.9), (0.9, 50, 0.8)])
def test_distribution_matches_the_analytic_one(temperature, top_k, top_p):
    from inference_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(1)
    V, n = 4000, 200_000
    row = torch.randn(V, device="cuda", generator=g) * 2.0
    want = _probs(row.cpu(), temperature, top_k, top_p)
    logits = row[None].expand(n, V).contiguous()
    toks = ops.sample_device(logits, temperature, top_k, top_p, torch.rand(n, device="cuda", generator=g))
    ops.check_status()
    got = torch.bincount(toks.cpu(), minlength=V).double() / n
    assert got[want == 0].sum() == 0                                        # nothing outside the kept set
    assert (got - want).abs().max().item() < 6e-3                           # ~5 sigma at the largest probabilities
    assert abs((got * torch.arange(V)).sum() - (want * torch.arange(V)).sum()) < 25
