"""Schedule builders and the per-step coefficient policy (gen-core/src/sampling.rs:61-650).

`StepCoeffs` expresses one sampler step as x' = a_x * x + a_out * model_out + a_noise * noise with the model fed
c_in * x at `timestep`; `FlowMatchPolicy` is the rectified-flow Euler step x += v * (sigma_next - sigma)."""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass


@dataclass(frozen=True)
class StepCoeffs:
    timestep: float
    c_in: float
    a_x: float
    a_out: float
    a_noise: float


class AlphaSchedule:
    def __init__(self, alphas_cumprod: list[float]):
        self.alphas_cumprod = alphas_cumprod

    @staticmethod
    def scaled_linear(num_train_timesteps: int = 1000, beta_start: float = 0.00085, beta_end: float = 0.012
                      ) -> "AlphaSchedule":
        n = num_train_timesteps
        a, b = math.sqrt(beta_start), math.sqrt(beta_end)
        acc, out = 1.0, []
        for i in range(n):
            t = 0.0 if n <= 1 else i / (n - 1)
            v = a + (b - a) * t
            acc *= 1.0 - v * v
            out.append(acc)
        return AlphaSchedule(out)

    def sigma_at(self, t: int) -> float:
        acp = self.alphas_cumprod[t]
        return math.sqrt((1.0 - acp) / acp)


def lcm_style_timesteps(num_train_timesteps: int, original_steps: int, num_steps: int) -> list[int]:
    original_steps, num_steps = max(1, original_steps), max(1, num_steps)
    k = num_train_timesteps // original_steps
    rev = [i * k - 1 for i in range(1, original_steps + 1)][::-1]
    return [rev[min(int(math.floor(len(rev) * j / num_steps)), len(rev) - 1)] for j in range(num_steps)]


def image_seq_len(width: int, height: int) -> int:
    return max(1, height // 16) * max(1, width // 16)


def compute_mu(seq_len: int, num_steps: int) -> float:
    """FLUX resolution-dependent schedule shift (empirical two-line fit in sequence length and step count)."""
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if seq_len > 4300:
        return a2 * seq_len + b2
    m_200 = a2 * seq_len + b2
    m_10 = a1 * seq_len + b1
    a = (m_200 - m_10) / 190.0
    b = m_200 - 200.0 * a
    return a * num_steps + b


def time_shift_exponential(mu: float, t: float) -> float:
    e = math.exp(mu)
    return e / (e + (1.0 / t - 1.0))


def build_flow_sigmas(num_steps: int, mu: float) -> list[float]:
    """linspace(1, 1/n, n) pushed through the exponential time shift, plus the terminal 0."""
    n = max(1, num_steps)
    start, end = 1.0, 1.0 / n
    out = []
    for i in range(n):
        t = start if n == 1 else start + (end - start) * i / (n - 1)
        out.append(time_shift_exponential(mu, t))
    out.append(0.0)
    return out


def flow_capture_plan(sigmas: list[float], capture_sigma: float | None) -> tuple[int, float] | None:
    """Earliest step whose sigma is at/below the ceiling: (number of schedule nodes to keep, that sigma)."""
    if capture_sigma is None or not math.isfinite(capture_sigma) or capture_sigma <= 0 or len(sigmas) < 2:
        return None
    for k in range(1, len(sigmas)):
        if sigmas[k] <= capture_sigma:
            return (k + 1, sigmas[k]) if sigmas[k] > 0 else None
    return None


def vp_sigma_from_edm(edm_sigma: float) -> float:
    if not math.isfinite(edm_sigma) or edm_sigma <= 0:
        return 0.0
    return edm_sigma / math.sqrt(1.0 + edm_sigma * edm_sigma)


class TimestepConvention(enum.Enum):
    SIGMA = "sigma"
    ONE_MINUS_SIGMA = "one_minus_sigma"


class FlowMatchPolicy:
    def __init__(self, sigmas: list[float], conv: TimestepConvention = TimestepConvention.SIGMA):
        assert len(sigmas) >= 2, "FlowMatchPolicy needs num_steps + 1 sigmas"
        self.sigmas, self.conv = list(sigmas), conv

    def num_steps(self) -> int:
        return len(self.sigmas) - 1

    def init_noise_scale(self) -> float:
        return 1.0

    def sigma(self, i: int) -> float:
        return self.sigmas[i]

    def coeffs(self, i: int) -> StepCoeffs:
        s = self.sigmas[i]
        t = s if self.conv is TimestepConvention.SIGMA else 1.0 - s
        return StepCoeffs(t, 1.0, 1.0, self.sigmas[i + 1] - s, 0.0)


def run_policy(policy, x, predict, noise=None):
    """Drives any step policy: x is scaled by init_noise_scale, then for every step
    x = a_x x + a_out predict(c_in x, timestep) + a_noise noise(i). Works on floats or tensors."""
    x = x * policy.init_noise_scale()
    for i in range(policy.num_steps()):
        c = policy.coeffs(i)
        out = predict(x * c.c_in, c.timestep)
        x = x * c.a_x + out * c.a_out
        if c.a_noise != 0.0:
            if noise is None:
                raise ValueError("this policy injects noise: pass noise(step)")
            x = x + noise(i) * c.a_noise
    return x


class LightningPolicy:
    """SDXL-Lightning: Euler over trailing-spaced timesteps (N - j N / steps, rounded, minus one), noise prediction,
    sigmas interpolated from the training table, terminal sigma 0 (gen-core/src/sampling.rs:449-520)."""

    def __init__(self, sched: AlphaSchedule, num_train_timesteps: int, num_steps: int):
        num_steps = max(1, num_steps)
        ratio = num_train_timesteps / num_steps
        self.timesteps = [float(round(num_train_timesteps - ratio * j) - 1) for j in range(num_steps)]
        full = [sched.sigma_at(t) for t in range(num_train_timesteps)]

        def interp(t: float) -> float:
            tt = min(max(t, 0.0), num_train_timesteps - 1)
            lo = int(math.floor(tt))
            hi = min(lo + 1, num_train_timesteps - 1)
            f = tt - lo
            return full[lo] * (1.0 - f) + full[hi] * f

        self.sigmas = [interp(t) for t in self.timesteps] + [0.0]

    def num_steps(self) -> int:
        return len(self.timesteps)

    def init_noise_scale(self) -> float:
        return max(self.sigmas)

    def sigma(self, i: int) -> float:
        return self.sigmas[i]

    def coeffs(self, i: int) -> StepCoeffs:
        s = self.sigmas[i]
        return StepCoeffs(self.timesteps[i], 1.0 / math.sqrt(s * s + 1.0), 1.0, self.sigmas[i + 1] - s, 0.0)


class LcmPolicy:
    """Latent consistency: the boundary-condition mix of x and the noise prediction gives the denoised sample, which
    every step but the last re-noises to the next timestep (gen-core/src/sampling.rs:522-600)."""

    def __init__(self, sched: AlphaSchedule, num_train_timesteps: int, original_inference_steps: int, num_steps: int,
                 timestep_scaling: float = 10.0):
        self.sched = sched
        self.timesteps = lcm_style_timesteps(num_train_timesteps, original_inference_steps, num_steps)
        self.timestep_scaling = timestep_scaling

    def num_steps(self) -> int:
        return len(self.timesteps)

    def init_noise_scale(self) -> float:
        return 1.0

    def sigma(self, i: int):
        return None

    def denoised_coeffs(self, i: int) -> StepCoeffs:
        t = self.timesteps[i]
        apt = self.sched.alphas_cumprod[t]
        bpt = 1.0 - apt
        st = t * self.timestep_scaling
        c_skip = 0.25 / (st * st + 0.25)
        c_out = st / math.sqrt(st * st + 0.25)
        return StepCoeffs(float(t), 1.0, c_out / math.sqrt(apt) + c_skip, -c_out * math.sqrt(bpt) / math.sqrt(apt), 0.0)

    def coeffs(self, i: int) -> StepCoeffs:
        det = self.denoised_coeffs(i)
        if i == len(self.timesteps) - 1:
            return det
        ap = self.sched.alphas_cumprod[self.timesteps[i + 1]]
        s = math.sqrt(ap)
        return StepCoeffs(det.timestep, 1.0, det.a_x * s, det.a_out * s, math.sqrt(1.0 - ap))


class TcdPolicy:
    """Trajectory consistency (Hyper-SD): each step jumps to the intermediate timestep s = floor((1 - eta) t_next)
    deterministically and, for eta > 0, re-noises from s up to t_next (gen-core/src/sampling.rs:602-700)."""

    def __init__(self, sched: AlphaSchedule, num_train_timesteps: int, original_inference_steps: int, num_steps: int,
                 eta: float = 0.3):
        self.sched, self.eta = sched, eta
        self.timesteps = lcm_style_timesteps(num_train_timesteps, original_inference_steps, num_steps)

    def num_steps(self) -> int:
        return len(self.timesteps)

    def init_noise_scale(self) -> float:
        return 1.0

    def sigma(self, i: int):
        return None

    def _s(self, i: int) -> int:
        prev_t = 0 if i == len(self.timesteps) - 1 else self.timesteps[i + 1]
        return int(math.floor((1.0 - self.eta) * prev_t))

    def pred_noised_coeffs(self, i: int) -> StepCoeffs:
        t = self.timesteps[i]
        acp = self.sched.alphas_cumprod
        apt, aps = acp[t], acp[self._s(i)]
        bpt, bps = 1.0 - apt, 1.0 - aps
        return StepCoeffs(float(t), 1.0, math.sqrt(aps / apt), math.sqrt(bps) - math.sqrt(aps) * math.sqrt(bpt) / math.sqrt(apt),
                          0.0)

    def coeffs(self, i: int) -> StepCoeffs:
        det = self.pred_noised_coeffs(i)
        if self.eta > 0.0 and i != len(self.timesteps) - 1:
            acp = self.sched.alphas_cumprod
            ratio = acp[self.timesteps[i + 1]] / acp[self._s(i)]
            r = math.sqrt(ratio)
            return StepCoeffs(det.timestep, 1.0, det.a_x * r, det.a_out * r, math.sqrt(max(0.0, 1.0 - ratio)))
        return det
