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


@pytest.mark.parametrize("T,N,K", [(1, 200, 256), (3, 512, 4096), (5, 300, 14336), (8, 130, 7168), (2, 33, 1024)])
def test_q4k_matvec_kernel_matches_reference_and_the_tensor_core_path(T, N, K):
    """Up to 8 tokens of Q4_K run the integer matrix-vector kernel (int8 activations per 32-block); splits = -1 keeps
    the dequantising tensor-core kernel. Both against CPU dequantisation + fp32 matmul."""
    from inference_b200 import ops
    from inference_b200.ops import quant

    g = torch.Generator().manual_seed(T * 7 + K)
    w = torch.randn(N, K, generator=g) * 0.05
    qw = quant.quantize_weight(w, "Q4_K").to("cuda")
    wref = quant.dequantize_reference(qw)
    a = (torch.randn(T, K, generator=g) * 0.5).bfloat16().cuda()
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16().cuda()
    ref = a.float().cpu() @ wref.t() + bias.float().cpu()
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    mv = quant.linear_quant(a, qw, bias=bias)
    tc = quant.linear_quant(a, qw, bias=bias, splits=-1)
    ops.check_status()
    assert (mv.float().cpu() - ref).abs().max().item() < tol
    assert (tc.float().cpu() - ref).abs().max().item() < tol
    assert not torch.equal(mv, tc) or T * N < 64          # two different kernels produced the two results
    # activations with a zero block and a large outlier block keep their per-block scales
    a2 = a.clone()
    a2[:, :32] = 0
    a2[:, 32:64] *= 40
    ref2 = a2.float().cpu() @ wref.t()
    out2 = quant.linear_quant(a2, qw)
    assert (out2.float().cpu() - ref2).abs().max().item() < 2e-2 * max(1.0, ref2.abs().max().item())


def test_large_token_count_uses_dense_path():
    from inference_b200.ops import quant

    w = torch.randn(512, 512) * 0.05
    qw = quant.quantize_weight(w, "Q8_0").to("cuda")
    a = (torch.randn(200, 512) * 0.5).bfloat16().cuda()
    out = quant.linear_quant(a, qw)
    ref = a.float().cpu() @ quant.dequantize_reference(qw).t()
    assert (out.float().cpu() - ref).abs().max().item() < 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("T,N,K", [(1, 256, 512), (16, 384, 1024), (64, 200, 256), (33, 3072, 3072)])
def test_nvfp4_gemm_and_dequant_match_cpu_container(T, N, K):
    """The device decode of E2M1 codes and swizzled E4M3 scales reproduces the container's dequantised values
    exactly (they are bf16-representable up to the scale product), and the fused GEMM matches fp32 matmul on them."""
    from inference_b200 import ops
    from inference_b200.ops import nvfp4 as nv

    g = torch.Generator().manual_seed(T + N)
    w = torch.randn(N, K, generator=g) * 0.05
    w[1, 3] = 1.5
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16().cuda()
    lin = nv.Nvfp4Linear(nv.Nvfp4Tensor.pack(w).to("cuda"), bias)
    ref_w = lin.t.dequantize()                                     # fp32 on the device, torch ops
    dense = lin.dense_bf16()
    ops.check_status()
    torch.testing.assert_close(dense.float(), ref_w.bfloat16().float(), rtol=1e-2, atol=1e-6)
    x = torch.randn(T, K, generator=g).bfloat16().cuda()
    y = lin(x)
    ops.check_status()
    ref = x.float() @ dense.float().t() + bias.float()             # the kernel multiplies exactly these bf16 weights
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    big = torch.randn(130, K, generator=g).bfloat16().cuda()       # more than 64 rows: expand + dense GEMM
    torch.testing.assert_close(lin(big).float(), big.float() @ dense.float().t() + bias.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("rows,cols,dtype", [(130, 80, torch.float32), (64, 4096, torch.bfloat16), (1, 16, torch.float32),
                                            (257, 3072, torch.float32)])
def test_nvfp4_device_quantiser_is_bit_identical_to_the_host_packer(rows, cols, dtype):
    from inference_b200 import ops
    from inference_b200.ops import nvfp4 as nv

    g = torch.Generator().manual_seed(rows + cols)
    x = (torch.randn(rows, cols, generator=g) * 0.3).to(dtype)
    x[0, 0] = 7.0                                           # an outlier fixes the tensor scale
    x[rows // 2, : min(32, cols)] = 0.0                     # all-zero blocks: scale byte 0, codes 0
    if cols >= 32:
        x[rows - 1, 16:32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25] * 2).to(dtype) * 0.01
    host = nv.Nvfp4Tensor.pack(x)
    dev = nv.quantize_on_device(x.cuda())
    ops.check_status()
    assert dev.global_scale == host.global_scale
    assert torch.equal(dev.scales.cpu(), host.scales)
    assert torch.equal(dev.packed.cpu(), host.packed)
    torch.testing.assert_close(nv.quantize_activations(x.cuda()).cpu().float(), host.dequantize().to(dtype).float())


@pytest.mark.parametrize("T,N,K", [(128, 128, 256), (300, 400, 512), (1000, 272, 1024), (65, 4096, 3072)])
def test_nvfp4_w4a4_tensor_core_gemm_matches_the_dequantised_product(T, N, K):
    """Both operands 4-bit in the tensor core: the result equals the fp32 product of the two dequantised NVFP4
    tensors (every partial product is exact in fp32; only the accumulation order differs)."""
    from inference_b200 import ops
    from inference_b200.ops import nvfp4 as nv

    g = torch.Generator().manual_seed(T + N + K)
    w = torch.randn(N, K, generator=g) * 0.05
    x = (torch.randn(T, K, generator=g) * 0.7).bfloat16()
    x[:, :16] *= 6.0                                              # one loud block per row: block scales matter
    wq = nv.Nvfp4Tensor.pack(w).to("cuda")
    bias = (torch.randn(N, generator=g) * 0.1).bfloat16().cuda()
    out = nv.gemm_w4a4(x.cuda(), wq, bias)
    ops.check_status()
    xq = nv.Nvfp4Tensor.pack(x.float())
    ref = xq.dequantize() @ wq.to("cpu").dequantize().t() + bias.float().cpu()
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 1e-2 * max(1.0, ref.abs().max().item()), err
    lin = nv.Nvfp4Linear(wq, bias, act_precision=nv.ActPrecision.W4A4)
    assert torch.equal(lin(x.cuda()), out)                       # the layer takes the same path above 64 rows
