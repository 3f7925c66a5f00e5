"""Host-side failure detection for multi-rank jobs, and the fault plan used to test it.

The reference is a single process (typed errors, cooperative cancellation, socket deadlines: core-llm/src/error.rs:11-40,
mlx-llm/server/src/main.rs:189-242); everything here is new. Device-side waits are bounded in the kernels themselves
(status words, `CollectiveTimeout`); this module covers what the host must notice *between* steps:

* `Heartbeat`: every rank publishes a monotonically increasing beat into the job's key-value store; `check()` before a
  collective step raises `RankFailure` naming the ranks whose beat is older than the deadline, so no kernel that waits
  on a dead peer is ever launched.
* `FaultPlan` (SWB_FAULT_PLAN or explicit): host-injected faults - a rank that stops beating / exits at a step, a
  dropped arrival on the host barrier, capability probes forced false (peer access, NVLS) to drive the library
  fallback, load errors at a named stage. Nothing in a plan touches a GPU.
* `guarded_step`: wraps one engine step: heartbeat check, the step, status check; on a typed failure it marks the
  communicator health (`healthy | degraded | failed`) and re-raises, so a scheduler can release the batch's KV blocks
  and re-queue the requests elsewhere."""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field

from ..contracts.errors import CollectiveTimeout, InferenceError


class RankFailure(InferenceError):
    def __init__(self, ranks: list[int], detail: str = ""):
        super().__init__(f"ranks {ranks} stopped responding{': ' + detail if detail else ''}")
        self.ranks = ranks


@dataclass
class FaultPlan:
    die_at_step: dict[int, int] = field(default_factory=dict)       # rank -> step at which it exits the job
    silent_at_step: dict[int, int] = field(default_factory=dict)    # rank -> step from which it stops beating
    skip_barrier: dict[int, int] = field(default_factory=dict)      # rank -> host-barrier index it does not join
    deny: set[str] = field(default_factory=set)                      # capability probes forced false: "peer", "nvls"
    fail_load_stage: str | None = None                                # raise LoadError at this stage name

    @staticmethod
    def from_env() -> "FaultPlan":
        raw = os.environ.get("SWB_FAULT_PLAN")
        if not raw:
            return FaultPlan()
        j = json.loads(raw)
        as_int = lambda d: {int(k): int(v) for k, v in (d or {}).items()}   # noqa: E731
        return FaultPlan(as_int(j.get("die_at_step")), as_int(j.get("silent_at_step")), as_int(j.get("skip_barrier")),
                         set(j.get("deny", [])), j.get("fail_load_stage"))

    def denies(self, capability: str) -> bool:
        return capability in self.deny

    def check_load_stage(self, stage: str) -> None:
        if self.fail_load_stage == stage:
            from ..contracts.errors import LoadError

            raise LoadError(f"injected load failure at stage '{stage}'")


class Heartbeat:
    """Beats live in a torch.distributed store (TCPStore / the process group's store): key `hb/<rank>` holds
    `<step>:<wall time>`."""

    def __init__(self, store, rank: int, world: int, deadline_s: float = 5.0, plan: FaultPlan | None = None,
                 clock=time.time):
        self.store, self.rank, self.world, self.deadline_s = store, rank, world, deadline_s
        self.plan = plan or FaultPlan()
        self.clock = clock
        self.step = 0
        self.beat()

    def beat(self) -> None:
        silent_from = self.plan.silent_at_step.get(self.rank)
        if silent_from is not None and self.step >= silent_from:
            return
        self.store.set(f"hb/{self.rank}", f"{self.step}:{self.clock():.3f}")

    def ages(self) -> dict[int, float]:
        now = self.clock()
        out = {}
        for r in range(self.world):
            try:
                raw = self.store.get(f"hb/{r}").decode()
                out[r] = now - float(raw.split(":")[1])
            except Exception:
                out[r] = float("inf")
        return out

    def check(self) -> None:
        """Raise RankFailure if any peer's last beat is older than the deadline."""
        late = [r for r, age in self.ages().items() if r != self.rank and age > self.deadline_s]
        if late:
            raise RankFailure(late, f"no heartbeat for more than {self.deadline_s:.1f} s")

    def advance(self) -> None:
        self.step += 1
        self.beat()


def host_barrier(store, name: str, rank: int, world: int, timeout_s: float, plan: FaultPlan | None = None,
                 index: int = 0) -> None:
    """A store-based barrier with a deadline (the host model of the device flag barrier): every rank adds 1 to a
    counter and polls until it reaches `world`. A rank whose plan says so never arrives; the others raise
    CollectiveTimeout naming how many arrived."""
    plan = plan or FaultPlan()
    key = f"bar/{name}/{index}"
    if plan.skip_barrier.get(rank) == index:
        return
    store.add(key, 1)
    t0 = time.time()
    while True:
        n = store.add(key, 0)
        if n >= world:
            return
        if time.time() - t0 > timeout_s:
            raise CollectiveTimeout(f"host barrier '{name}'#{index}: {n} of {world} ranks arrived within {timeout_s} s")
        time.sleep(0.005)


def guarded_step(comm, heartbeat: Heartbeat | None, step_fn, status_fn=None):
    """Run one step with failure detection around it; updates comm.health and re-raises typed failures."""
    try:
        if heartbeat is not None:
            heartbeat.check()
        out = step_fn()
        if status_fn is not None:
            status_fn()
        if heartbeat is not None:
            heartbeat.advance()
        return out
    except RankFailure:
        comm.health = "failed"
        raise
    except CollectiveTimeout:
        comm.health = "failed" if comm.fused is None else "degraded"
        raise
