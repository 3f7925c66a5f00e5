"""Model-sampling parameterisations: how a network output at noise level sigma maps to the denoised estimate
(gen-core/src/sampling/model_sampling.rs:22-371). Flow (rectified flow / CONST), Discrete (eps / v over the
scaled-linear DDPM table) and EDM (continuous v-prediction)."""
from __future__ import annotations

import abc
import enum
import math

from .policy import AlphaSchedule, TimestepConvention


class PredictionType(enum.Enum):
    EPS = "eps"
    V = "v"
    FLOW = "flow"


class ModelSampling(abc.ABC):
    @abc.abstractmethod
    def prediction(self) -> PredictionType: ...
    @abc.abstractmethod
    def sigma_min(self) -> float: ...
    @abc.abstractmethod
    def sigma_max(self) -> float: ...
    @abc.abstractmethod
    def input_scale(self, sigma: float) -> float: ...
    @abc.abstractmethod
    def denoised_coeffs(self, sigma: float) -> tuple[float, float]:
        """(k_x, k_out): x0 = k_x * x + k_out * model_out."""
    @abc.abstractmethod
    def timestep(self, sigma: float) -> float: ...
    @abc.abstractmethod
    def sigma(self, timestep: float) -> float: ...

    def noise_scaling_coeffs(self, sigma: float) -> tuple[float, float]:
        return sigma, 1.0

    def num_timesteps(self) -> int:
        return 1000

    def sigma_table(self) -> list[float]:
        n = self.num_timesteps()
        lo, hi = self.timestep(self.sigma_min()), self.timestep(self.sigma_max())
        return [self.sigma(lo + (hi - lo) * (0.0 if n <= 1 else i / (n - 1))) for i in range(n)]


def denoise(ops, ms: ModelSampling, x, sigma: float, run_model):
    s = ms.input_scale(sigma)
    x_in = x if s == 1.0 else ops.scale(x, s)
    raw = run_model(x_in, ms.timestep(sigma))
    k_x, k_out = ms.denoised_coeffs(sigma)
    return ops.axpy(k_x, x, k_out, raw)


def cfgpp_denoise(ops, ms: ModelSampling, x, sigma: float, run_model_pair):
    s = ms.input_scale(sigma)
    x_in = x if s == 1.0 else ops.scale(x, s)
    guided, uncond = run_model_pair(x_in, ms.timestep(sigma))
    k_x, k_out = ms.denoised_coeffs(sigma)
    return ops.axpy(k_x, x, k_out, guided), ops.axpy(k_x, x, k_out, uncond)


class FlowModelSampling(ModelSampling):
    def __init__(self, conv: TimestepConvention = TimestepConvention.SIGMA, mu: float = 0.0):
        self.conv, self.mu = conv, mu

    def prediction(self):
        return PredictionType.FLOW

    def sigma_min(self):
        return 1.0 / self.num_timesteps()

    def sigma_max(self):
        return 1.0

    def input_scale(self, sigma):
        return 1.0

    def denoised_coeffs(self, sigma):
        return 1.0, -sigma        # x0 = x - sigma * v

    def noise_scaling_coeffs(self, sigma):
        return sigma, 1.0 - sigma  # x_sigma = sigma * noise + (1 - sigma) * x0

    def timestep(self, sigma):
        return sigma if self.conv is TimestepConvention.SIGMA else 1.0 - sigma

    def sigma(self, timestep):
        t = timestep if self.conv is TimestepConvention.SIGMA else 1.0 - timestep
        if self.mu == 0.0 or t <= 0.0:
            return max(t, 0.0)
        e = math.exp(self.mu)
        return e / (e + (1.0 / t - 1.0))


class DiscreteModelSampling(ModelSampling):
    """eps- or v-prediction over the DDPM scaled-linear table; timestep <-> sigma by log-sigma interpolation."""

    def __init__(self, prediction: PredictionType = PredictionType.EPS, schedule: AlphaSchedule | None = None):
        assert prediction in (PredictionType.EPS, PredictionType.V)
        self._pred = prediction
        sch = schedule or AlphaSchedule.scaled_linear()
        self._sigmas = [sch.sigma_at(t) for t in range(len(sch.alphas_cumprod))]
        self._log = [math.log(s) for s in self._sigmas]

    def prediction(self):
        return self._pred

    def num_timesteps(self):
        return len(self._sigmas)

    def sigma_min(self):
        return self._sigmas[0]

    def sigma_max(self):
        return self._sigmas[-1]

    def input_scale(self, sigma):
        return 1.0 / math.sqrt(sigma * sigma + 1.0)

    def denoised_coeffs(self, sigma):
        if self._pred is PredictionType.EPS:
            return 1.0, -sigma
        d = sigma * sigma + 1.0
        return 1.0 / d, -sigma / math.sqrt(d)

    def timestep(self, sigma):
        ls = math.log(max(sigma, 1e-12))
        lo, hi = 0, len(self._log) - 1
        if ls <= self._log[0]:
            return 0.0
        if ls >= self._log[-1]:
            return float(hi)
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self._log[mid] <= ls:
                lo = mid
            else:
                hi = mid
        w = (ls - self._log[lo]) / (self._log[hi] - self._log[lo])
        return lo + w

    def sigma(self, timestep):
        t = min(max(timestep, 0.0), len(self._log) - 1.0)
        lo = int(math.floor(t))
        hi = min(lo + 1, len(self._log) - 1)
        w = t - lo
        return math.exp((1.0 - w) * self._log[lo] + w * self._log[hi])

    def sigma_table(self):
        return list(self._sigmas)


class EdmModelSampling(ModelSampling):
    """Continuous EDM v-prediction (sigma_data preconditioning), timestep = 0.25 * ln(sigma)."""

    def __init__(self, sigma_min: float = 0.002, sigma_max: float = 120.0, sigma_data: float = 1.0):
        self._min, self._max, self.sigma_data = sigma_min, sigma_max, sigma_data

    def prediction(self):
        return PredictionType.V

    def sigma_min(self):
        return self._min

    def sigma_max(self):
        return self._max

    def input_scale(self, sigma):
        return 1.0 / math.sqrt(sigma * sigma + self.sigma_data ** 2)

    def denoised_coeffs(self, sigma):
        sd2 = self.sigma_data ** 2
        d = sigma * sigma + sd2
        return sd2 / d, -sigma * self.sigma_data / math.sqrt(d)

    def timestep(self, sigma):
        return 0.25 * math.log(max(sigma, 1e-12))

    def sigma(self, timestep):
        return math.exp(timestep / 0.25)
