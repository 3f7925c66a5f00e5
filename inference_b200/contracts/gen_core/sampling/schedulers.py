"""Sigma schedulers (gen-core/src/sampling/schedulers.rs:22-246): normal, simple, karras, exponential,
sgm_uniform, beta, ddim_uniform, beta57. Each returns steps + 1 descending sigmas ending in 0 (beta may drop
duplicate nodes). The inverse Beta CDF is computed here (regularised incomplete beta by continued fraction,
inverted by bisection) so no SciPy dependency is needed."""
from __future__ import annotations

import math

from .model_sampling import ModelSampling

SCHEDULERS = ("normal", "simple", "karras", "exponential", "sgm_uniform", "beta", "ddim_uniform", "beta57")


def _table_range(ms: ModelSampling) -> tuple[float, float]:
    table = ms.sigma_table()
    hi = table[-1] if table else 1.0
    lo = next((s for s in table if s > 0.0), max(hi * 1e-3, 1e-4))
    return lo, hi


def karras_sigmas(n: int, sigma_min: float, sigma_max: float, rho: float = 7.0) -> list[float]:
    n = max(1, n)
    mn, mx = max(sigma_min, 0.0) ** (1.0 / rho), sigma_max ** (1.0 / rho)
    return [(mx + (0.0 if n == 1 else i / (n - 1)) * (mn - mx)) ** rho for i in range(n)] + [0.0]


def exponential_sigmas(n: int, sigma_min: float, sigma_max: float) -> list[float]:
    n = max(1, n)
    lmin, lmax = math.log(max(sigma_min, 1e-12)), math.log(max(sigma_max, 1e-12))
    return [math.exp(lmax + (lmin - lmax) * (0.0 if n == 1 else i / (n - 1))) for i in range(n)] + [0.0]


def normal_sigmas(ms: ModelSampling, steps: int, sgm: bool) -> list[float]:
    steps = max(1, steps)
    start, end = ms.timestep(ms.sigma_max()), ms.timestep(ms.sigma_min())
    out = []
    for i in range(steps):
        f = i / steps if sgm else (0.0 if steps == 1 else i / (steps - 1))
        out.append(ms.sigma(start + (end - start) * f))
    return out + [0.0]


def simple_sigmas(ms: ModelSampling, steps: int) -> list[float]:
    steps = max(1, steps)
    table = ms.sigma_table()
    n = len(table)
    if n == 0:
        return [0.0]
    ss = n / steps
    return [table[min(max(n - (1 + int(x * ss)), 0), n - 1)] for x in range(steps)] + [0.0]


def ddim_uniform_sigmas(ms: ModelSampling, steps: int) -> list[float]:
    steps = max(1, steps)
    table = ms.sigma_table()
    n = len(table)
    if n <= 1:
        return [0.0]
    if abs(table[1]) < 1e-5:
        steps += 1
    ss = max(1, n // steps)
    sigs = [table[x] for x in range(1, n, ss)]
    return sigs[::-1] + [0.0]


def _ln_gamma(x: float) -> float:
    return math.lgamma(x)


def _betacf(a: float, b: float, x: float) -> float:
    tiny = 1e-300
    qab, qap, qam = a + b, a + 1.0, a - 1.0
    c, d = 1.0, 1.0 - qab * x / qap
    d = 1.0 / (d if abs(d) > tiny else tiny)
    h = d
    for m in range(1, 300):
        m2 = 2 * m
        aa = m * (b - m) * x / ((qam + m2) * (a + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        h *= d * c
        aa = -(a + m) * (qab + m) * x / ((a + m2) * (qap + m2))
        d = 1.0 + aa * d
        d = 1.0 / (d if abs(d) > tiny else tiny)
        c = 1.0 + aa / c
        c = c if abs(c) > tiny else tiny
        delta = d * c
        h *= delta
        if abs(delta - 1.0) < 3e-16:
            break
    return h


def _betainc(a: float, b: float, x: float) -> float:
    if x <= 0.0:
        return 0.0
    if x >= 1.0:
        return 1.0
    bt = math.exp(_ln_gamma(a + b) - _ln_gamma(a) - _ln_gamma(b) + a * math.log(x) + b * math.log(1.0 - x))
    if x < (a + 1.0) / (a + b + 2.0):
        return bt * _betacf(a, b, x) / a
    return 1.0 - bt * _betacf(b, a, 1.0 - x) / b


def beta_ppf(q: float, a: float, b: float) -> float:
    """Inverse of the regularised incomplete beta function (scipy.stats.beta.ppf)."""
    if q <= 0.0:
        return 0.0
    if q >= 1.0:
        return 1.0
    lo, hi = 0.0, 1.0
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if _betainc(a, b, mid) < q:
            lo = mid
        else:
            hi = mid
        if hi - lo < 1e-15:
            break
    return 0.5 * (lo + hi)


def beta_sigmas(ms: ModelSampling, steps: int, alpha: float, beta: float) -> list[float]:
    steps = max(1, steps)
    table = ms.sigma_table()
    n = len(table)
    if n == 0:
        return [0.0]
    total = max(n - 1, 0)
    sigs, last = [], -1
    for i in range(steps):
        t = int(round(beta_ppf(1.0 - i / steps, alpha, beta) * total))
        if t != last:
            sigs.append(table[min(max(t, 0), n - 1)])
        last = t
    return sigs + [0.0]


def schedule_sigmas(name: str, ms: ModelSampling, steps: int) -> list[float]:
    steps = max(1, steps)
    if name == "karras":
        return karras_sigmas(steps, *_table_range(ms), 7.0)
    if name == "exponential":
        return exponential_sigmas(steps, *_table_range(ms))
    if name == "normal":
        return normal_sigmas(ms, steps, False)
    if name == "sgm_uniform":
        return normal_sigmas(ms, steps, True)
    if name == "simple":
        return simple_sigmas(ms, steps)
    if name == "ddim_uniform":
        return ddim_uniform_sigmas(ms, steps)
    if name == "beta":
        return beta_sigmas(ms, steps, 0.6, 0.6)
    if name == "beta57":
        return beta_sigmas(ms, steps, 0.5, 0.7)
    raise KeyError(f"unknown scheduler {name!r}; known: {SCHEDULERS}")
