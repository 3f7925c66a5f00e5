"""Failure detection on the host: heartbeats, a rank that leaves between steps, a dropped barrier arrival, forced
capability fallbacks and injected load errors. Runs gloo CPU ranks as child processes; touches no GPU."""
import json
import os
import subprocess
import sys

import pytest

from inference_b200.contracts.errors import LoadError
from inference_b200.parallel.health import FaultPlan, Heartbeat, RankFailure

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode, world, port, plan=None):
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="")
        if plan:
            env["SWB_FAULT_PLAN"] = json.dumps(plan)
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_health_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\nTIMEOUT"
        outs.append((p.returncode, out))
    return outs


def test_healthy_job_stays_healthy():
    outs = _run("healthy", 2, 29711)
    assert all(rc == 0 and f"RANK{r}_HEALTHY" in out for r, (rc, out) in enumerate(outs)), outs


def test_rank_that_leaves_between_steps_is_detected_before_the_next_launch():
    outs = _run("die", 3, 29721, {"die_at_step": {"1": 2}})
    assert "RANK1_EXIT step=2" in outs[1][1]
    for r in (0, 2):
        rc, out = outs[r]
        assert rc == 0 and f"RANK{r}_DETECTED" in out and "ranks=[1]" in out, out


def test_dropped_barrier_arrival_times_out_with_a_typed_error():
    outs = _run("barrier", 2, 29731, {"skip_barrier": {"1": 1}})
    assert "RANK0_BARRIER timeout" in outs[0][1] and "RANK1_BARRIER passed" in outs[1][1], outs


def test_heartbeat_and_fault_plan_units(monkeypatch):
    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]
    now = [100.0]
    s = Store()
    plan = FaultPlan(silent_at_step={1: 2})
    a = Heartbeat(s, 0, 2, deadline_s=1.0, plan=plan, clock=lambda: now[0])
    b = Heartbeat(s, 1, 2, deadline_s=1.0, plan=plan, clock=lambda: now[0])
    for _ in range(3):
        now[0] += 0.5
        a.advance()
        b.advance()            # rank 1 goes silent from step 2 on
        a.check() if b.step < 3 else None
    now[0] += 0.8
    a.beat()
    with pytest.raises(RankFailure) as e:
        a.check()
    assert e.value.ranks == [1]
    monkeypatch.setenv("SWB_FAULT_PLAN", json.dumps({"deny": ["peer", "nvls"], "fail_load_stage": "transformer"}))
    p = FaultPlan.from_env()
    assert p.denies("peer") and p.denies("nvls") and not p.denies("tma")
    p.check_load_stage("vae")
    with pytest.raises(LoadError):
        p.check_load_stage("transformer")
