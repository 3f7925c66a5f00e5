"""Backend-neutral sampler framework: schedules, model-sampling parameterisations, solvers, CFG++
(parity: gen-core/src/sampling.rs and gen-core/src/sampling/*.rs)."""
from .latent_ops import CpuLatentOps, LatentOps, TorchLatentOps  # noqa: F401
from .model_sampling import (DiscreteModelSampling, EdmModelSampling, FlowModelSampling, ModelSampling,  # noqa: F401
                             PredictionType, TimestepConvention, cfgpp_denoise, denoise)
from .policy import (AlphaSchedule, FlowMatchPolicy, LcmPolicy, LightningPolicy, StepCoeffs, TcdPolicy, run_policy, build_flow_sigmas, compute_mu,  # noqa: F401
                     flow_capture_plan, image_seq_len, lcm_style_timesteps, time_shift_exponential,
                     vp_sigma_from_edm)
from .schedulers import SCHEDULERS, beta_ppf, exponential_sigmas, karras_sigmas, schedule_sigmas  # noqa: F401
from .solvers import SOLVERS, Euler, get_solver  # noqa: F401
from .scm import ScmScheduler, run_scm_sampler  # noqa: F401
