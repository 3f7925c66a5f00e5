"""Continuous-time consistency (sCM / TrigFlow) few-step sampler (parity: candle-gen/src/sampler.rs:462-625, the
`ScmScheduler` + `run_scm_sampler` pair used by SANA-Sprint).

Time runs on the quarter circle: x_t = cos(t) x_0 + sin(t) z with t from pi / 2 to 0. The network was trained in
flow coordinates, so each step converts: scm_t = sin t / (cos t + sin t), the input is scaled by
sqrt(scm_t^2 + (1 - scm_t)^2) / sigma_data, and the raw output is mapped back to the TrigFlow velocity before the
consistency step x_0 = cos(s) x - sin(s) F; every step but the last re-noises to the next time."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

from .latent_ops import LatentOps

SCM_MAX_TIMESTEP = math.pi / 2
SCM_INTERMEDIATE_TIMESTEP = 1.3
SCM_SIGMA_DATA = 0.5


@dataclass
class ScmScheduler:
    timesteps: list[float]
    sigma_data: float = SCM_SIGMA_DATA

    @staticmethod
    def new(num_steps: int, max_t: float = SCM_MAX_TIMESTEP, mid_t: float = SCM_INTERMEDIATE_TIMESTEP) -> "ScmScheduler":
        """Two steps use the trained intermediate time 1.3; any other count is a linear ramp from max_t to 0."""
        if num_steps == 2:
            return ScmScheduler([max_t, mid_t, 0.0])
        n = max(1, num_steps)
        return ScmScheduler([max_t * (1.0 - i / n) for i in range(n + 1)])

    @property
    def num_steps(self) -> int:
        return max(0, len(self.timesteps) - 1)

    def scm_timestep(self, i: int) -> float:
        t = self.timesteps[i]
        s, c = math.sin(t), math.cos(t)
        return s / (c + s)

    def input_scale(self, i: int) -> float:
        st = self.scm_timestep(i)
        return math.sqrt(st * st + (1.0 - st) * (1.0 - st))


def run_scm_sampler(ops: LatentOps, sched: ScmScheduler, latents, seed: int, predict: Callable,
                    on_step: Callable[[int, int], None] = lambda i, n: None):
    """latents: unit-variance noise. predict(x_in, scm_t) -> raw network output. Returns the denoised latent (data
    scale). on_step(current, total) is called before each evaluation (and may raise to cancel)."""
    sd = sched.sigma_data
    n = sched.num_steps
    single = n <= 1
    x = ops.scale(latents, sd)
    denoised = x
    for i in range(n):
        on_step(i + 1, max(1, n))
        s, t_next = sched.timesteps[i], sched.timesteps[i + 1]
        scm_t, in_scale = sched.scm_timestep(i), sched.input_scale(i)
        x_in = ops.scale(x, in_scale / sd)
        raw = predict(x_in, scm_t)
        a = 1.0 - 2.0 * scm_t
        b = 1.0 - 2.0 * scm_t + 2.0 * scm_t * scm_t
        out = ops.scale(ops.axpy(a, x_in, b, raw), sd / in_scale)
        denoised = ops.axpy(math.cos(s), x, -math.sin(s), out)
        if single:
            x = denoised
        else:
            noise = ops.scale(ops.randn_like(x, seed, i), sd)
            x = ops.axpy(math.cos(t_next), denoised, math.sin(t_next), noise)
    return ops.scale(denoised, 1.0 / sd)
