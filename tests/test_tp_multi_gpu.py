"""Tensor-parallel equivalence on 2+ GPUs (TP=k == TP=1 oracle; fused peer-memory all-reduce == NCCL baseline).
Runs the ranks as child processes; skipped on boxes with a single GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, mode, port, worker="_tp_worker.py", marker="TP_WORKER_OK", extra_env=None):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, worker), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and marker in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("mode", ["fused", "nccl"])
def test_sequence_parallel_dit_2gpu(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, mode, 29551 if mode == "fused" else 29552, "_sp_worker.py", "SP_WORKER_OK", {"SWB_SP": mode})


def test_sequence_parallel_dit_4gpu():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _run(4, "fused", 29553, "_sp_worker.py", "SP_WORKER_OK", {"SWB_SP": "fused"})


@pytest.mark.parametrize("mode", ["fused", "nccl"])
def test_tp2(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, mode, 29541 if mode == "fused" else 29542)


def test_tp4_fused():
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    _run(4, "fused", 29543)


def test_tp8_fused():
    if torch.cuda.device_count() < 8:
        pytest.skip("needs 8 GPUs")
    _run(8, "fused", 29544)


def test_bounded_flag_wait_times_out_without_faulting():
    """A wait on a flag nothing sets gives up after the (shortened) budget, reports it, and the context survives."""
    import ctypes

    from inference_b200 import ops
    from inference_b200._native import kernels

    L = kernels()
    L.swb_status_clear()
    L.swb_set_wait_limit_ns(20_000_000)  # 20 ms
    try:
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        res = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        rc = L.swb_flag_wait(flag.data_ptr(), 5, res.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert res.item() == 0
        st = ops.device_status()
        assert st[0] == 3 and st[1] == 2000
        L.swb_status_clear()
        flag.fill_(9)
        L.swb_flag_wait(flag.data_ptr(), 5, res.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert res.item() == 1 and ops.device_status()[0] == 0
        x = torch.ones(4, device="cuda")
        assert x.sum().item() == 4.0
    finally:
        L.swb_set_wait_limit_ns(2_000_000_000)
        L.swb_status_clear()
