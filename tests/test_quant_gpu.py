"""Weight-only quantised GEMM kernels against CPU dequantisation + fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", ["Q4_K", "Q8_0", "AFFINE4", "AFFINE8"])
@pytest.mark.parametrize("T,N,K,splits", [(1, 256, 512, 0), (8, 1000, 1024, 0), (64, 384, 2048, 3), (33, 128, 256, 1)])
def test_gemm_quant_matches_reference(fmt, T, N, K, splits):
    from inference_b200 import ops
    from inference_b200.ops import quant

    g = torch.Generator().manual_seed(T * 131 + N)
    w = torch.randn(N, K, generator=g) * 0.05
    qw = quant.quantize_weight(w, fmt).to("cuda")
    wref = quant.dequantize_reference(qw)                       # fp32 [N, K] from plain CPU math
    dense = quant.dequantize(qw)
    assert (dense.float().cpu() - wref).abs().max().item() <= 4e-3 * max(1.0, wref.abs().max().item())
    a = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16().cuda()
    for rep in range(2):                                         # second call reuses the workspace counters
        out = quant.linear_quant(a, qw, bias=bias, splits=splits)
        ops.check_status()
        ref = a.float().cpu() @ wref.t() + bias.float().cpu()
        err = (out.float().cpu() - ref).abs().max().item()
        assert err < 2e-2 * max(1.0, ref.abs().max().item()), (fmt, rep, err)


def test_large_token_count_uses_dense_path():
    from inference_b200.ops import quant

    w = torch.randn(512, 512) * 0.05
    qw = quant.quantize_weight(w, "Q8_0").to("cuda")
    a = (torch.randn(200, 512) * 0.5).bfloat16().cuda()
    out = quant.linear_quant(a, qw)
    ref = a.float().cpu() @ quant.dequantize_reference(qw).t()
    assert (out.float().cpu() - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())
