"""swb_argmax_static (the entry point that brings its own scratch) against swb_argmax, through the C symbol."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from inference_b200._native import kernels

    fn = kernels().swb_argmax_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _call(fn, logits, allow=None, want_vals=False):
    rows, V = logits.shape
    ids = torch.full((rows,), -1, dtype=torch.int64, device=logits.device)
    vals = torch.zeros(rows, dtype=torch.float32, device=logits.device) if want_vals else None
    rc = fn(logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0, logits.stride(0), rows, V,
            allow.data_ptr() if allow is not None else None, ids.data_ptr(),
            vals.data_ptr() if vals is not None else None, torch.cuda.current_stream().cuda_stream)
    return rc, ids, vals


@pytest.mark.parametrize("rows,V,dtype", [(1, 128256, torch.bfloat16), (64, 128256, torch.float32),
                                          (7, 32000, torch.bfloat16), (300, 20000, torch.float32),
                                          (5, 1000, torch.bfloat16)])
def test_matches_existing_entry_point_twice(rows, V, dtype):
    from inference_b200 import ops

    fn = _symbol()
    g = torch.Generator(device="cuda").manual_seed(rows * 7919 + V)
    for call in range(2):   # the second call reuses the array the first one left behind
        logits = torch.randn(rows, V, generator=g, device="cuda").to(dtype)
        if call == 1:
            logits[:, V // 3] = logits.max() + 1  # ties across rows' chunks resolve to this index unless beaten
            logits[0, 5] = logits[0, V // 3]       # exact tie: lowest index wins
        rc, ids, vals = _call(fn, logits, want_vals=True)
        assert rc == 0
        ref = ops.argmax(logits)
        torch.cuda.synchronize()
        assert torch.equal(ids, ref)
        assert torch.allclose(vals, logits.float().gather(1, ref[:, None])[:, 0], rtol=0, atol=0)


@pytest.mark.parametrize("rows,V,dtype", [(3, 128256, torch.float32), (40, 50000, torch.float32), (2, 777, torch.float32)])
def test_matches_torch_argmax_on_tie_free_rows(rows, V, dtype):
    """An independent oracle: distinct values per row (a shuffled ramp), so torch.argmax has one right answer."""
    fn = _symbol()
    g = torch.Generator(device="cuda").manual_seed(V + rows)
    ramp = torch.arange(V, device="cuda", dtype=torch.float32) * 1e-3 - 20.0
    logits = torch.stack([ramp[torch.randperm(V, generator=g, device="cuda")] for _ in range(rows)]).to(dtype)
    rc, ids, vals = _call(fn, logits, want_vals=True)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(ids, torch.argmax(logits, dim=-1))
    assert torch.equal(vals, logits.max(dim=-1).values.float())


def test_allow_mask_and_strided_rows():
    from inference_b200 import ops

    fn = _symbol()
    big = torch.randn(9, 40000 + 64, device="cuda")
    logits = big[:, :40000]                      # row stride larger than V
    allow = (torch.rand(40000, device="cuda") < 0.3).to(torch.uint8)
    for _ in range(2):
        rc, ids, _ = _call(fn, logits, allow=allow)
        assert rc == 0
        assert torch.equal(ids, ops.argmax(logits, allow_mask=allow))
        big.copy_(torch.randn_like(big))


def test_rejects_sizes_beyond_the_limit(capfd):
    fn = _symbol()
    logits = torch.zeros(2, 64, device="cuda")
    ids = torch.zeros(2, dtype=torch.int64, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert fn(logits.data_ptr(), 1, 64, 1025, 64, None, ids.data_ptr(), None, s) == -20
    assert fn(logits.data_ptr(), 1, 64, 2, 0, None, ids.data_ptr(), None, s) == -20
    assert fn(None, 1, 64, 2, 64, None, ids.data_ptr(), None, s) == -22
    assert fn(logits.data_ptr(), 1, 64, 0, 64, None, ids.data_ptr(), None, s) == 0
    assert "outside the supported range" in capfd.readouterr().err
    rc, out, _ = _call(fn, torch.eye(2, 64, device="cuda"))   # still usable after the refusals
    assert rc == 0 and out.tolist() == [0, 1]
