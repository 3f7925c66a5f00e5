"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, w, bias, residual, act):
    y = a.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "silu":
        y = torch.nn.functional.silu(y)
    elif act == "gelu_tanh":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual.float()
    return y


def _check(T, N, K, *, mode=-1, block_n=0, ctas=0, bias=False, residual=False, act=None, out_dtype=torch.bfloat16):
    from inference_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(T * 7919 + N * 31 + K)
    a = (torch.randn(T, K, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    b = (torch.randn(N, device="cuda", generator=g) * 0.1).bfloat16() if bias else None
    r = (torch.randn(T, N, device="cuda", generator=g) * 0.5).bfloat16() if residual else None
    y = ops.gemm_bf16(a, w, bias=b, residual=r, act=act, mode=mode, block_n=block_n, ctas=ctas,
                      out_dtype=out_dtype)
    ops.check_status()
    ref = _ref(a, w, b, r, act)
    err = (y.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert err / scale < tol, f"T={T} N={N} K={K} mode={mode} bn={block_n} ctas={ctas}: err {err} scale {scale}"
    return y


@pytest.mark.parametrize("T", [1, 5, 16, 33, 64, 128, 200, 256])
def test_swapped_small_tokens(T):
    _check(T, 512, 256)
    _check(T, 384, 1024, bias=True, residual=True)


@pytest.mark.parametrize("ctas", [-1, 3, 7, 20, 148])
def test_stream_k_deterministic(ctas):
    y0 = _check(8, 1024, 2048, mode=1, ctas=ctas, bias=True, act="silu")
    y1 = _check(8, 1024, 2048, mode=1, ctas=ctas, bias=True, act="silu")
    assert torch.equal(y0, y1)
    _check(300, 640, 1024, mode=0, ctas=ctas, residual=True)


@pytest.mark.parametrize("shape", [(300, 256, 128), (512, 1024, 512), (1000, 776, 328), (129, 4096, 4096)])
@pytest.mark.parametrize("block_n", [0, 64, 128])
def test_tokens_as_m(shape, block_n):
    T, N, K = shape
    _check(T, N, K, mode=0, block_n=block_n)
    _check(T, N, K, mode=0, block_n=block_n, bias=True, residual=True, act="gelu_tanh")


def test_fp32_out_and_ragged_edges():
    _check(77, 1000, 264, mode=0, out_dtype=torch.float32)
    _check(7, 1000, 264, mode=1, out_dtype=torch.float32, bias=True)
    _check(40, 136, 72, mode=1)
    _check(260, 136, 72)


def test_llama_shapes():
    for T in (1, 8, 64):
        _check(T, 6144, 4096)
        _check(T, 4096, 14336, residual=True)
    _check(1024, 6144, 4096)
    _check(1024, 4096, 14336, residual=True)


def test_strided_views():
    from inference_b200 import ops

    a = (torch.randn(48, 1024, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(256, 512, device="cuda") * 0.05).bfloat16()
    y = ops.gemm_bf16(a[:, 512:], w)
    ref = a[:, 512:].float() @ w.float().t()
    assert (y.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item()


@pytest.mark.parametrize("cluster", [1, 2, 3, 5, 6, 8])
@pytest.mark.parametrize("T", [1, 7, 16, 31, 64])
def test_cluster_split_k_decode(T, cluster):
    y0 = _check(T, 1024, 2048, mode=2, ctas=cluster, bias=True, residual=True, act="silu")
    y1 = _check(T, 1024, 2048, mode=2, ctas=cluster, bias=True, residual=True, act="silu")
    assert torch.equal(y0, y1)
    _check(T, 1000, 1096, mode=2, ctas=cluster, out_dtype=torch.float32)


@pytest.mark.parametrize("N,K", [(512, 256), (2816, 2048), (200, 320)])
def test_grouped_gemm_matches_per_group_matmul(N, K):
    """Each 128-row tile multiplies the weight group its table entry names; skipped tiles stay untouched."""
    from inference_b200 import ops

    G = 5
    g = torch.Generator(device="cuda").manual_seed(0)
    w = (torch.randn(G, N, K, device="cuda", generator=g) * 0.05).bfloat16()
    table = torch.tensor([3, 0, -1, 4, 4, 1, -1, 2], dtype=torch.int32, device="cuda")
    R = table.numel() * 128
    a = torch.randn(R, K, device="cuda", generator=g).bfloat16()
    out = torch.full((R, N), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm_bf16_grouped(a, w, table, out=out)
    ops.check_status()
    for i, e in enumerate(table.tolist()):
        rows = slice(i * 128, (i + 1) * 128)
        if e < 0:
            assert torch.all(out[rows] == 7.0)
            continue
        ref = a[rows].float() @ w[e].float().t()
        torch.testing.assert_close(out[rows].float(), ref, rtol=2e-2, atol=2e-2)
    act = ops.gemm_bf16_grouped(a, w, table, act="silu")
    ref = torch.nn.functional.silu(a[:128].float() @ w[3].float().t())
    torch.testing.assert_close(act[:128].float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,F,K,act", [(1, 256, 1024, "silu"), (64, 14336, 4096, "silu"), (17, 1000, 768, "gelu_tanh"),
                                       (200, 512, 1024, "silu")])
def test_gated_projection_pairs(T, F, K, act):
    """Gate-up projection with interleaved (gate, up) rows: fused epilogue (decode sizes) and GEMM + paired
    activation kernel (larger) both equal act(x Wg^T) * (x Wu^T)."""
    from inference_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(T + F)
    wg = (torch.randn(F, K, device="cuda", generator=g) * 0.03).bfloat16()
    wu = (torch.randn(F, K, device="cuda", generator=g) * 0.03).bfloat16()
    x = torch.randn(T, K, device="cuda", generator=g).bfloat16()
    pairs = torch.stack([wg, wu], dim=1).reshape(2 * F, K).contiguous()
    y = ops.linear_gated(x, pairs, act)
    ops.check_status()
    gate, up = x.float() @ wg.float().t(), x.float() @ wu.float().t()
    fn = torch.nn.functional.silu if act == "silu" else (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
    torch.testing.assert_close(y.float(), fn(gate) * up, rtol=3e-2, atol=3e-2)
    assert ops.gated_fused(T, 2 * F, K) == (T <= 64)
