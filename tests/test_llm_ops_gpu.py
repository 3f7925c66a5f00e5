"""Fused LLM glue kernels and attention against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rope_tables(max_pos, rot_dim, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().cuda().contiguous(), ang.sin().cuda().contiguous()


def test_rmsnorm_and_residual():
    from inference_b200 import ops

    for T, H in ((1, 4096), (7, 256), (33, 8192), (5, 3072), (3, 1024)):
        x = torch.randn(T, H, device="cuda").bfloat16()
        r = torch.randn(T, H, device="cuda").bfloat16()
        w = (torch.randn(H, device="cuda") * 0.1 + 1).bfloat16()
        y = ops.rmsnorm(x, w, 1e-5)
        xf = x.float()
        ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
        r2 = r.clone()
        y2 = ops.rmsnorm(x, w, 1e-5, residual=r2)
        s = (x.float() + r.float()).bfloat16()
        assert torch.equal(r2, s)
        sf = s.float()
        ref2 = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        assert torch.allclose(y2.float(), ref2, atol=3e-2, rtol=2e-2)


def test_layernorm_mod_and_gated_residual():
    from inference_b200 import ops

    B, S, H = 2, 37, 3072
    x = torch.randn(B, S, H, device="cuda").bfloat16()
    sc = (torch.randn(B, H, device="cuda") * 0.2).bfloat16()
    sh = (torch.randn(B, H, device="cuda") * 0.2).bfloat16()
    y = ops.layernorm_mod(x, scale=sc, shift=sh, rows_per_batch=S, eps=1e-6)
    ref = torch.nn.functional.layer_norm(x.float(), (H,), eps=1e-6) * (1 + sc.float()[:, None]) + sh.float()[:, None]
    assert torch.allclose(y.float(), ref, atol=4e-2, rtol=2e-2)
    b = torch.randn(B, S, H, device="cuda").bfloat16()
    z = ops.gated_residual(x, b, sc, rows_per_batch=S)
    refz = x.float() + sc.float()[:, None] * b.float()
    assert torch.allclose(z.float(), refz, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("D,rot", [(128, 128), (64, 64), (128, 64), (96, 32)])
def test_rope_kv_write(interleaved, D, rot):
    from inference_b200 import ops

    T, Hq, Hkv, bs, nblk = 19, 4, 2, 16, 8
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(nblk * bs, device="cuda")[:T].to(torch.int64)
    cos, sin = _rope_tables(512, rot)
    kc = torch.zeros(nblk, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    ref = qkv.float().reshape(T, Hq + 2 * Hkv, D).clone()
    c = cos[pos.long()][:, None, :]
    s = sin[pos.long()][:, None, :]
    qk = ref[:, : Hq + Hkv, :rot]
    if interleaved:
        x0, x1 = qk[..., 0::2], qk[..., 1::2]
        rot_out = torch.stack([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1).flatten(-2)
    else:
        x0, x1 = qk[..., : rot // 2], qk[..., rot // 2:]
        rot_out = torch.cat([x0 * c - x1 * s, x1 * c + x0 * s], dim=-1)
    ref[:, : Hq + Hkv, :rot] = rot_out
    ops.rope_kv_write(qkv, pos, slots, cos, sin, kc, vc, Hq, Hkv, D, rot_dim=rot, interleaved=interleaved,
                      block_size=bs)
    got = qkv.float().reshape(T, Hq + 2 * Hkv, D)
    assert torch.allclose(got[:, :Hq], ref[:, :Hq], atol=3e-2, rtol=2e-2)
    blk, off = slots // bs, slots % bs
    kgot = kc[blk, :, off].float()
    vgot = vc[blk, :, off].float()
    assert torch.allclose(kgot, ref[:, Hq:Hq + Hkv], atol=3e-2, rtol=2e-2)
    assert torch.allclose(vgot, ref[:, Hq + Hkv:], atol=1e-6)


def test_qk_norm_rope():
    from inference_b200 import ops

    T, Hq, Hkv, D = 5, 4, 2, 128
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    ref = qkv.float().reshape(T, -1, D).clone()
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    cos, sin = _rope_tables(64, D)
    qw = (torch.rand(D, device="cuda") + 0.5).bfloat16()
    kw = (torch.rand(D, device="cuda") + 0.5).bfloat16()
    ops.rope_kv_write(qkv, pos, None, cos, sin, None, None, Hq, Hkv, D, q_norm=qw, k_norm=kw, norm_eps=1e-6)

    def nrm(x, w):
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).bfloat16().float()

    q = nrm(ref[:, :Hq], qw)
    c, s = cos[pos.long()][:, None], sin[pos.long()][:, None]
    q = torch.cat([q[..., :64] * c - q[..., 64:] * s, q[..., 64:] * c + q[..., :64] * s], -1)
    got = qkv.float().reshape(T, -1, D)[:, :Hq]
    assert torch.allclose(got, q, atol=4e-2, rtol=2e-2)


def test_gated_act_embedding_argmax():
    from inference_b200 import ops

    gu = torch.randn(9, 2 * 1376, device="cuda").bfloat16()
    y = ops.gated_act_mul(gu)
    ref = torch.nn.functional.silu(gu[:, :1376].float()) * gu[:, 1376:].float()
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    table = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (4, 7), device="cuda")
    e = ops.embedding(ids, table)
    assert torch.equal(e, table[ids.reshape(-1)])
    logits = torch.randn(6, 128256, device="cuda")
    logits[2, 77] = 50.0
    logits[2, 99000] = 50.0
    am = ops.argmax(logits)
    assert torch.equal(am, logits.argmax(-1)) or am[2].item() == 77
    assert am[2].item() == 77
    allow = torch.zeros(128256, dtype=torch.uint8, device="cuda")
    allow[1000:2000] = 1
    am2 = ops.argmax(logits.bfloat16(), allow)
    assert torch.equal(am2, logits.bfloat16()[:, 1000:2000].float().argmax(-1) + 1000)
    t = torch.tensor([[5, 6, 7, 8, 9], [5, 1, 7, 8, 9]], device="cuda")
    d = torch.tensor([[5, 6, 7, 0], [5, 6, 7, 8]], device="cuda")
    n, nxt = ops.spec_verify_greedy(t, d)
    assert n.tolist() == [3, 1] and nxt.tolist() == [8, 1]


def _ref_attn(q, k, v, scale, causal):
    # q [Sq, Hq, D], k/v [Skv, Hkv, D]
    Sq, Hq, D = q.shape
    Skv, Hkv, _ = k.shape
    G = Hq // Hkv
    kf = k.float().repeat_interleave(G, dim=1)
    vf = v.float().repeat_interleave(G, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None]
        j = torch.arange(Skv, device=q.device)[None, :]
        s = s.masked_fill(j > i + (Skv - Sq), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf).reshape(Sq, Hq * D)


def _build_paged(kv_lens, Hkv, D, bs=16, extra=3):
    nblk_per = [(n + bs - 1) // bs for n in kv_lens]
    total = sum(nblk_per) + extra
    perm = torch.randperm(total).tolist()
    kc = torch.randn(total, Hkv, bs, D, device="cuda").bfloat16()
    vc = torch.randn(total, Hkv, bs, D, device="cuda").bfloat16()
    maxb = max(nblk_per)
    table = torch.zeros(len(kv_lens), maxb, dtype=torch.int32)
    ks, vs = [], []
    it = iter(perm)
    for i, n in enumerate(kv_lens):
        ids = [next(it) for _ in range(nblk_per[i])]
        table[i, : len(ids)] = torch.tensor(ids, dtype=torch.int32)
        kk = kc[ids].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:n]
        vv = vc[ids].permute(0, 2, 1, 3).reshape(-1, Hkv, D)[:n]
        ks.append(kk)
        vs.append(vv)
    return kc, vc, table.cuda(), ks, vs


@pytest.mark.parametrize("Hq,Hkv", [(8, 2), (4, 4)])
def test_paged_prefill(Hq, Hkv):
    from inference_b200 import ops

    D = 128
    q_lens = [70, 1, 129, 64]
    kv_lens = [70, 40, 200, 64]
    kc, vc, table, ks, vs = _build_paged(kv_lens, Hkv, D)
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda").bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    out = ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=max(q_lens), scale=scale, causal=True)
    o = 0
    for i, n in enumerate(q_lens):
        ref = _ref_attn(q[o:o + n], ks[i], vs[i], scale, True)
        err = (out[o:o + n].float() - ref).abs().max().item()
        assert err < 3e-2, (i, err)
        o += n


@pytest.mark.parametrize("bs", [8, 16, 32, 128])
def test_paged_prefill_tcgen05_against_reference_and_mma_sync(bs, monkeypatch):
    """Prefill on top of earlier context, pages read through TMA: several page sizes, contexts that end mid page and
    mid tile, one sequence with no earlier context, uniform query lengths without cu_q, and the non-causal form."""
    from inference_b200 import ops

    D, Hq, Hkv = 128, 8, 2
    q_lens = [300, 17, 128, 256]
    kv_lens = [1500, 401, 128, 257]
    kc, vc, table, ks, vs = _build_paged(kv_lens, Hkv, D, bs=bs)
    T = sum(q_lens)
    q = torch.randn(T, Hq, D, device="cuda").bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    for causal in (True, False):
        out = ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=max(q_lens), scale=scale, causal=causal)
        o = 0
        for i, n in enumerate(q_lens):
            ref = _ref_attn(q[o:o + n], ks[i], vs[i], scale, causal)
            err = (out[o:o + n].float() - ref).abs().max().item()
            assert err < 3e-2, (causal, i, err)
            o += n
    if bs == 16:
        monkeypatch.setenv("SWB_PAGED_PREFILL", "legacy")
        old = ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=max(q_lens), scale=scale, causal=True)
        monkeypatch.setenv("SWB_PAGED_PREFILL", "tcgen05")
        new = ops.paged_attention(q, kc, vc, table, kvl, cu_q=cu, max_q_len=max(q_lens), scale=scale, causal=True)
        assert (old.float() - new.float()).abs().max().item() < 3e-2
    # uniform query lengths, no cu_q
    kv2 = [200, 136, 264]
    kc, vc, table, ks, vs = _build_paged(kv2, Hkv, D, bs=bs)
    q = torch.randn(3 * 136, Hq, D, device="cuda").bfloat16()
    out = ops.paged_attention(q, kc, vc, table, torch.tensor(kv2, dtype=torch.int32, device="cuda"), cu_q=None, max_q_len=136,
                              scale=scale, causal=True)
    for i in range(3):
        ref = _ref_attn(q[i * 136:(i + 1) * 136], ks[i], vs[i], scale, True)
        assert (out[i * 136:(i + 1) * 136].float() - ref).abs().max().item() < 3e-2, i


@pytest.mark.parametrize("use_tma", [True, False])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("q_len", [1, 3])
def test_paged_decode(splits, q_len, use_tma):
    from inference_b200 import ops

    D, Hq, Hkv = 128, 16, 4
    kv_lens = [1 + q_len, 63, 64, 65, 500, 1300]
    kc, vc, table, ks, vs = _build_paged(kv_lens, Hkv, D)
    B = len(kv_lens)
    q = torch.randn(B * q_len, Hq, D, device="cuda").bfloat16()
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(D)
    out = ops.paged_attention(q, kc, vc, table, kvl, cu_q=None, max_q_len=q_len, scale=scale, causal=True,
                              decode=True, num_splits=splits, use_tma=use_tma)
    ops.check_status()
    for i in range(B):
        ref = _ref_attn(q[i * q_len:(i + 1) * q_len], ks[i], vs[i], scale, True)
        err = (out[i * q_len:(i + 1) * q_len].float() - ref).abs().max().item()
        assert err < 3e-2, (i, err)


def test_dense_attention_noncausal():
    from inference_b200 import ops

    B, S, H, D = 2, 333, 6, 128
    qkv = torch.randn(B, S, 3, H, D, device="cuda").bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    scale = 1 / math.sqrt(D)
    out = ops.dense_attention(q, k, v, scale=scale)
    for b in range(B):
        ref = _ref_attn(q[b], k[b], v[b], scale, False)
        assert (out[b].float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("B,Sq,Skv,Hq,Hkv,qmul", [(1, 4608, 4608, 4, 4, 1.0), (2, 300, 1000, 8, 2, 1.0),
                                                   (1, 1024, 2048, 2, 1, 6.0), (1, 129, 257, 2, 2, 1.0),
                                                   (1, 256, 128, 1, 1, 12.0)])
def test_dense_attention_tcgen05(B, Sq, Skv, Hq, Hkv, qmul):
    """tcgen05 kernel against fp32 math and against the mma.sync kernel; qmul > 1 spreads the logits so that the
    running maximum keeps growing and the lazy accumulator rescale is exercised."""
    from inference_b200 import ops
    from inference_b200.ops.attention import set_dense_impl

    g = torch.Generator(device="cuda").manual_seed(Sq * 31 + Skv)
    q = (torch.randn(B, Sq, Hq, 128, device="cuda", generator=g) * qmul).bfloat16()
    k = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(B, Skv, Hkv, 128, device="cuda", generator=g).bfloat16()
    if qmul > 1:   # keys later in the sequence score higher on average
        k = (k.float() + q.float().mean(1, keepdim=True)[:, :, :Hkv] * torch.linspace(
            0, 0.05, Skv, device="cuda")[None, :, None, None]).bfloat16()
    scale = 1 / math.sqrt(128)
    out = ops.dense_attention(q, k, v, scale=scale)
    ops.check_status()
    set_dense_impl(True)
    try:
        legacy = ops.dense_attention(q, k, v, scale=scale)
    finally:
        set_dense_impl(False)
    from inference_b200._native import kernels

    forced = []
    try:
        for tiles in (1, 2):          # both schedules: one query tile per CTA, two with softmax / MMA overlap
            kernels().swb_attn_dense_set_tiles(tiles)
            forced.append(ops.dense_attention(q, k, v, scale=scale))
            ops.check_status()
    finally:
        kernels().swb_attn_dense_set_tiles(0)
    for b in range(B):
        ref = _ref_attn(q[b], k[b], v[b], scale, False)
        err = (out[b].float() - ref).abs().max().item()
        assert err < 3e-2, (b, err)
        assert (out[b].float() - legacy[b].float()).abs().max().item() < 3e-2
        for f in forced:
            assert (f[b].float() - ref).abs().max().item() < 3e-2


@pytest.mark.parametrize("lens,Hq,Hkv", [([300, 17, 1024, 129], 8, 2), ([64], 4, 4), ([1000, 1000], 2, 1)])
def test_varlen_causal_attention_tcgen05(lens, Hq, Hkv):
    """Packed fresh-prefill attention straight from a QKV buffer (strided views) against fp32 causal attention."""
    from inference_b200 import ops

    T = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(T)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * 128, device="cuda", generator=g).bfloat16()
    q = qkv[:, : Hq * 128].view(T, Hq, 128)
    k = qkv[:, Hq * 128:(Hq + Hkv) * 128].view(T, Hkv, 128)
    v = qkv[:, (Hq + Hkv) * 128:].view(T, Hkv, 128)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    scale = 1 / math.sqrt(128)
    out = ops.varlen_causal_attention(q, k, v, cu, max(lens), scale=scale)
    ops.check_status()
    lo = 0
    for n in lens:
        ref = _ref_attn(q[lo:lo + n], k[lo:lo + n], v[lo:lo + n], scale, True)
        err = (out[lo:lo + n].float() - ref).abs().max().item()
        assert err < 3e-2, (n, err)
        lo += n
