"""gloo CPU ranks for the failure-detection tests (launched as child processes; no GPU involved)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    import torch.distributed as dist

    from inference_b200.contracts.errors import CollectiveTimeout
    from inference_b200.parallel import init_distributed
    from inference_b200.parallel.health import FaultPlan, Heartbeat, RankFailure, guarded_step, host_barrier

    mode = sys.argv[1]
    comm = init_distributed(backend="gloo", timeout_s=20)
    rank, world = comm.rank, comm.world
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0, wait_for_workers=True)
    plan = FaultPlan.from_env()
    hb = Heartbeat(store, rank, world, deadline_s=1.2, plan=plan)    # generous: the ranks share a busy host
    if mode in ("die", "healthy"):
        # processes start (and import) at different speeds: line the ranks up, then publish a fresh beat, so that the
        # first check measures time since this point and not since the fastest rank came up
        host_barrier(store, "start", rank, world, 60.0, plan, index=99)
        hb.beat()
    if mode == "die":
        # every rank steps; rank 1 leaves between steps (no collective in flight); the others notice before launching
        detected = None
        for step in range(24):
            if plan.die_at_step.get(rank) == step:
                print(f"RANK{rank}_EXIT step={step}", flush=True)
                os._exit(0)
            try:
                def work():
                    t = torch.ones(4) * (rank + 1)
                    alive = [r for r in range(world) if plan.die_at_step.get(r, 1 << 30) > step]
                    if len(alive) == world:
                        dist.all_reduce(t)
                    return t
                guarded_step(comm, hb, work)
            except RankFailure as e:
                detected = (step, e.ranks)
                break
            time.sleep(0.25)
        assert detected is not None and detected[1] == [1], detected
        assert comm.health == "failed"
        print(f"RANK{rank}_DETECTED step={detected[0]} ranks={detected[1]}", flush=True)
    elif mode == "barrier":
        host_barrier(store, "warm", rank, world, 5.0, plan, index=0)
        try:
            host_barrier(store, "step", rank, world, 1.0, plan, index=1)
            outcome = "passed"
        except CollectiveTimeout as e:
            outcome = "timeout:" + str(e)
        if plan.skip_barrier.get(rank) == 1:
            assert outcome == "passed"            # the rank that skipped never waited
        else:
            assert outcome.startswith("timeout") and f"{world - 1} of {world}" in outcome, outcome
        print(f"RANK{rank}_BARRIER {outcome[:7]}", flush=True)
    elif mode == "healthy":
        for _ in range(3):
            guarded_step(comm, hb, lambda: dist.all_reduce(torch.ones(2)))
        assert comm.health == "healthy" and max(hb.ages().values()) < 1.2
        print(f"RANK{rank}_HEALTHY", flush=True)
    # rank 0 hosts the store: it leaves after every surviving rank has finished with it
    store.add("finished", 1)
    survivors = world - len(plan.die_at_step)
    t0 = time.time()
    while rank == 0 and store.add("finished", 0) < survivors and time.time() - t0 < 10.0:
        time.sleep(0.02)
    os._exit(0)


if __name__ == "__main__":
    main()
