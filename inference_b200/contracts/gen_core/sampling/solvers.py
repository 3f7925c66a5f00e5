"""Samplers in the unified sigma space written once over LatentOps (gen-core/src/sampling/unified.rs:29-104 and
solvers.rs:53-708): euler, euler_ancestral, heun, dpmpp_2m, dpmpp_sde, uni_pc, lcm, ddim, er_sde, dpmpp_2m_sde.
`denoise(x, sigma)` returns the denoised estimate x0; lambda = -ln(sigma)."""
from __future__ import annotations

import math


def _to_d(ops, x, sigma, x0):
    return ops.scale(ops.sub(x, x0), 1.0 / sigma)


def ancestral_step(s_from: float, s_to: float, eta: float = 1.0) -> tuple[float, float]:
    """Split a step into a deterministic descent to sigma_down and fresh noise sigma_up (k-diffusion)."""
    if not eta:
        return s_to, 0.0
    up = min(s_to, eta * math.sqrt(max(s_to ** 2 * (s_from ** 2 - s_to ** 2) / s_from ** 2, 0.0)))
    return math.sqrt(max(s_to ** 2 - up ** 2, 0.0)), up


class Sampler:
    name = "base"

    def sample(self, ops, ms, denoise, x, sigmas, seed: int = 0):
        raise NotImplementedError


class Euler(Sampler):
    name = "euler"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        for i in range(len(sigmas) - 1):
            s = sigmas[i]
            x0 = denoise(x, s)
            if s == 0.0:
                x = x0
                continue
            x = ops.axpy(1.0, x, sigmas[i + 1] - s, _to_d(ops, x, s, x0))
        return x


class EulerAncestral(Sampler):
    name = "euler_ancestral"

    def __init__(self, eta: float = 1.0):
        self.eta = eta

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        for i in range(len(sigmas) - 1):
            s = sigmas[i]
            x0 = denoise(x, s)
            if s == 0.0:
                x = x0
                continue
            sd, su = ancestral_step(s, sigmas[i + 1], self.eta)
            x = ops.axpy(1.0, x, sd - s, _to_d(ops, x, s, x0))
            if su > 0.0:
                x = ops.axpy(1.0, x, su, ops.randn_like(x, seed, i))
        return x


class Heun(Sampler):
    name = "heun"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s)
            if s == 0.0:
                x = x0
                continue
            d = _to_d(ops, x, s, x0)
            dt = sn - s
            if sn == 0.0:
                x = ops.axpy(1.0, x, dt, d)
            else:
                x2 = ops.axpy(1.0, x, dt, d)
                d2 = _to_d(ops, x2, sn, denoise(x2, sn))
                x = ops.axpy(1.0, x, dt, ops.axpy(0.5, d, 0.5, d2))
        return x


class Dpmpp2m(Sampler):
    name = "dpmpp_2m"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        old = None
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s)
            if s == 0.0 or sn == 0.0:
                x = x0
                old = x0
                continue
            t, tn = -math.log(s), -math.log(sn)
            h = tn - t
            if old is None:
                d = x0
            else:
                h_last = t - (-math.log(sigmas[i - 1]))
                r = h_last / h
                d = ops.axpy(1.0 + 1.0 / (2.0 * r), x0, -1.0 / (2.0 * r), old)
            x = ops.axpy(sn / s, x, -math.expm1(-h), d)
            old = x0
        return x


class DpmppSde(Sampler):
    name = "dpmpp_sde"

    def __init__(self, eta: float = 1.0, r: float = 0.5):
        self.eta, self.r = eta, r

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s)
            if s == 0.0:
                x = x0
                continue
            if sn == 0.0:
                x = ops.axpy(1.0, x, sn - s, _to_d(ops, x, s, x0))
                continue
            t, tn = -math.log(s), -math.log(sn)
            h = tn - t
            sm = math.exp(-(t + h * self.r))
            fac = 1.0 / (2.0 * self.r)
            sd, su = ancestral_step(s, sm, self.eta)
            x2 = ops.axpy(sd / s, x, -math.expm1(-(-math.log(sd) - t)) if sd > 0 else 1.0, x0)
            if su > 0:
                x2 = ops.axpy(1.0, x2, su, ops.randn_like(x, seed, 2 * i))
            x0_2 = denoise(x2, sm)
            sd, su = ancestral_step(s, sn, self.eta)
            d = ops.axpy(1.0 - fac, x0, fac, x0_2)
            x = ops.axpy(sd / s, x, -math.expm1(-(-math.log(sd) - t)) if sd > 0 else 1.0, d)
            if su > 0:
                x = ops.axpy(1.0, x, su, ops.randn_like(x, seed, 2 * i + 1))
        return x


class UniPc(Sampler):
    """UniPC (bh2) of order 2 in data-prediction form: a DPM-Solver++(2M) style predictor followed by the
    unified corrector that reuses the model evaluation made at the new point."""
    name = "uni_pc"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        prev = None          # (lambda, x0) of the previous node
        cur0 = None
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s) if cur0 is None else cur0
            cur0 = None
            if s == 0.0 or sn == 0.0:
                x = x0
                prev = None
                continue
            lam, lam_n = -math.log(s), -math.log(sn)
            h = lam_n - lam
            hh = -h
            h_phi_1 = math.expm1(hh)
            b_h = math.expm1(hh)
            if prev is None:
                x_pred = ops.axpy(sn / s, x, -h_phi_1, x0)
                d1 = None
            else:
                r = (prev[0] - lam) / h
                d1 = ops.scale(ops.sub(prev[1], x0), 1.0 / r)
                x_pred = ops.axpy(1.0, ops.axpy(sn / s, x, -h_phi_1, x0), -0.5 * b_h, d1)
            x0_n = denoise(x_pred, sn)
            # corrector (order = predictor order + 1, bh2 coefficients)
            h_phi_k = h_phi_1 / hh - 1.0
            d1_t = ops.sub(x0_n, x0)
            if d1 is None:
                x = ops.axpy(1.0, ops.axpy(sn / s, x, -h_phi_1, x0), -b_h * 0.5, d1_t)
            else:
                # two-point corrector: solve the 2x2 system for (rho_prev, rho_new)
                rk = (prev[0] - lam) / h
                b1 = h_phi_k * 1.0 / b_h
                h_phi_k2 = h_phi_k / hh - 0.5
                b2 = h_phi_k2 * 2.0 / b_h
                det = rk - 1.0
                rho_p = (b1 - b2) / det if abs(det) > 1e-12 else 0.0
                rho_c = b1 - rho_p
                if abs(det) <= 1e-12:
                    rho_c = 0.5
                x = ops.axpy(sn / s, x, -h_phi_1, x0)
                x = ops.axpy(1.0, x, -b_h * rho_p, d1)
                x = ops.axpy(1.0, x, -b_h * rho_c, d1_t)
            prev = (lam, x0)
            cur0 = None   # the corrected point differs from x_pred: re-evaluate at the next step
        return x


class Lcm(Sampler):
    name = "lcm"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        for i in range(len(sigmas) - 1):
            x0 = denoise(x, sigmas[i])
            x = x0
            sn = sigmas[i + 1]
            if sn > 0.0:
                k_noise, k_x0 = ms.noise_scaling_coeffs(sn)
                x = ops.axpy(k_x0, x0, k_noise, ops.randn_like(x0, seed, i))
        return x


class Ddim(Sampler):
    """Deterministic DDIM (eta = 0): in sigma space identical to the Euler step along d = (x - x0) / sigma."""
    name = "ddim"

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        return Euler().sample(ops, ms, denoise, x, sigmas, seed)


def _er_noise_scaler(lam: float) -> float:
    return lam * (math.exp(lam ** 0.3) + 10.0)


class ErSde(Sampler):
    name = "er_sde"

    def __init__(self, s_noise: float = 1.0, max_stage: int = 3):
        self.s_noise, self.max_stage = s_noise, max_stage

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        num_int = 200.0
        point = [i / num_int for i in range(int(num_int))]
        old = old_d = None
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s)
            stage = min(self.max_stage, i + 1)
            if sn == 0.0 or s == 0.0:
                x = x0
            else:
                er_s, er_t = _er_noise_scaler(s), _er_noise_scaler(sn)
                r = er_t / er_s
                x = ops.axpy(r, x, 1.0 - r, x0)
                if stage >= 2 and old is not None:
                    dt = sn - s
                    lam_step = [-dt * p + sn for p in point] if False else [sn + (s - sn) * p for p in point]
                    s_int = sum(1.0 / _er_noise_scaler(l) for l in lam_step) * ((s - sn) / num_int)
                    d = ops.scale(ops.sub(x0, old), 1.0 / (s - sigmas[i - 1]))
                    x = ops.axpy(1.0, x, (dt + s_int * er_t), d)
                    if stage >= 3 and old_d is not None:
                        s_u = sum((l - s) / _er_noise_scaler(l) for l in lam_step) * ((s - sn) / num_int)
                        dd = ops.scale(ops.sub(d, old_d), 2.0 / (s - sigmas[i - 2]))
                        x = ops.axpy(1.0, x, (dt ** 2 / 2.0 + s_u * er_t), dd)
                    old_d = d
                if self.s_noise > 0:
                    var = max(sn ** 2 - (s * r) ** 2, 0.0)
                    if var > 0:
                        x = ops.axpy(1.0, x, self.s_noise * math.sqrt(var), ops.randn_like(x, seed, i))
            old = x0
        return x


class Dpmpp2mSde(Sampler):
    name = "dpmpp_2m_sde"

    def __init__(self, eta: float = 1.0, s_noise: float = 1.0):
        self.eta, self.s_noise = eta, s_noise

    def sample(self, ops, ms, denoise, x, sigmas, seed=0):
        old, h_last = None, None
        for i in range(len(sigmas) - 1):
            s, sn = sigmas[i], sigmas[i + 1]
            x0 = denoise(x, s)
            if s == 0.0 or sn == 0.0:
                x = x0
            else:
                t, tn = -math.log(s), -math.log(sn)
                h = tn - t
                eta_h = self.eta * h
                x = ops.axpy(sn / s * math.exp(-eta_h), x, -math.expm1(-h - eta_h), x0)
                if old is not None:
                    r = h_last / h
                    x = ops.axpy(1.0, x, 0.5 * (-math.expm1(-h - eta_h)) / r, ops.sub(x0, old))
                if self.eta:
                    x = ops.axpy(1.0, x, sn * math.sqrt(max(-math.expm1(-2.0 * eta_h), 0.0)) * self.s_noise,
                                 ops.randn_like(x, seed, i))
                h_last = h
            old = x0
        return x


SOLVERS = {c.name: c for c in (Euler, EulerAncestral, Heun, Dpmpp2m, DpmppSde, UniPc, Lcm, Ddim, ErSde, Dpmpp2mSde)}


def get_solver(name: str) -> Sampler:
    if name not in SOLVERS:
        raise KeyError(f"unknown sampler {name!r}; known: {sorted(SOLVERS)}")
    return SOLVERS[name]()
