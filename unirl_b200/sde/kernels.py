"""SDE / ODE step strategies for flow-matching samplers.

Every stochastic strategy reduces one transition to three per-sample coefficients

    mean = a_x · x + a_v · v            x' = mean + s · ε

plus a log-prob form (Gaussian with std ``s``, or CPS's un-normalised ``−(x'−mean)²``).  That
reduction is what the fused sm_100a kernel consumes (``ops/sde_step``: one pass over the latent
produces ``x'``, ``mean`` and the per-sample mean log-prob); the PyTorch path below is the fp32
oracle the kernel is tested against and the CPU fallback.

Math parity: ``unirl/sde/kernels.py`` — ``StepStrategy.denoise`` ``:43-112``, dtype round-trip +
mean-reduced log-prob ``:154-177``, Flow ``:185-236``, CPS ``:239-279``, Dance ``:282-333``,
DPM-Solver-2 ``:341-515``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import ClassVar, List, Optional, Tuple

import torch

LOGP_GAUSSIAN = 0
LOGP_NEG_SQ = 1
_HALF_LOG_2PI = 0.5 * math.log(2.0 * math.pi)


@dataclass
class TransitionCoeffs:
    """Per-sample coefficients of one transition (tensors broadcastable against the latent)."""

    a_x: torch.Tensor
    a_v: torch.Tensor
    noise_std: torch.Tensor
    logp_mode: int = LOGP_GAUSSIAN


def _expand(sigma: torch.Tensor, ndim: int) -> torch.Tensor:
    sigma = sigma.float()
    if sigma.dim() == 0:
        sigma = sigma.unsqueeze(0)
    while sigma.dim() < ndim:
        sigma = sigma.unsqueeze(-1)
    return sigma


class StepStrategy:
    """One denoising transition.  ``denoise`` returns ``(x', log_prob | None, mean | None)``."""

    canonical_name: ClassVar[str] = "ode"
    is_stochastic: ClassVar[bool] = False

    def reset(self) -> None:
        pass

    def init_schedule(self, sigmas: torch.Tensor) -> None:
        pass

    def coeffs(self, sigma: torch.Tensor, sigma_next: torch.Tensor, eta: float, sigma_max: float) -> TransitionCoeffs:
        """Euler flow-matching ODE: ``x' = x + (σ' − σ)·v``."""
        one = torch.ones_like(sigma)
        return TransitionCoeffs(one, sigma_next - sigma, torch.zeros_like(sigma))

    def denoise(self, noise_pred: torch.Tensor, sample: torch.Tensor, sigma: torch.Tensor, sigma_next: torch.Tensor, *,
                eta: float = 1.0, prev_sample: Optional[torch.Tensor] = None, sigma_max: float = 0.99, step_index: int = 0,
                noise: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None,
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        """fp32 transition.  ``prev_sample=None`` ⇒ sample (draw or use ``noise``); else score the given transition.

        The new sample is round-tripped through the input dtype *before* the log-prob is taken so
        that replay from stored (lower precision) latents reproduces the rollout's log-prob.
        """
        in_dtype = sample.dtype
        v, x = noise_pred.float(), sample.float()
        s, s_next = _expand(sigma, x.dim()), _expand(sigma_next, x.dim())
        c = self.coeffs(s, s_next, float(eta), float(sigma_max))
        mean = c.a_x * x + c.a_v * v
        if not self.is_stochastic:
            return mean, None, None
        if prev_sample is None:
            if noise is None:
                noise = torch.randn(v.shape, dtype=v.dtype, device=v.device, generator=generator)
            prev = mean + c.noise_std * noise.float()
        else:
            prev = prev_sample.float()
        if eta < 1e-7:
            return prev, None, mean
        prev = prev.to(in_dtype).float()
        return prev, self.log_prob(prev, mean, c).mean(dim=tuple(range(1, x.dim()))), mean

    @staticmethod
    def log_prob(prev: torch.Tensor, mean: torch.Tensor, c: TransitionCoeffs) -> torch.Tensor:
        d2 = (prev.detach() - mean) ** 2
        if c.logp_mode == LOGP_NEG_SQ:
            return -d2
        return -d2 / (2 * c.noise_std**2) - torch.log(c.noise_std) - _HALF_LOG_2PI


class SDEStrategy(StepStrategy):
    is_stochastic: ClassVar[bool] = True


def _flow_mean_coeffs(std: torch.Tensor, sigma: torch.Tensor, dt: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    return 1 + std**2 / (2 * sigma) * dt, (1 + std**2 * (1 - sigma) / (2 * sigma)) * dt


class FlowSDEStrategy(SDEStrategy):
    """FlowGRPO SDE: ``std = sqrt(σ/(1−σ̃))·η`` with ``σ̃ = σ_max`` where ``σ == 1``; noise std ``std·sqrt(−dt)``."""

    canonical_name: ClassVar[str] = "flow"

    def __init__(self, *, config: Optional["FlowSpec"] = None) -> None:
        pass

    def coeffs(self, sigma, sigma_next, eta, sigma_max):
        dt = sigma_next - sigma
        std = torch.sqrt(sigma / (1 - torch.where(sigma == 1, torch.full_like(sigma, sigma_max), sigma))) * eta
        a_x, a_v = _flow_mean_coeffs(std, sigma, dt)
        return TransitionCoeffs(a_x, a_v, std * torch.sqrt(-dt))


class DanceSDEStrategy(SDEStrategy):
    """DanceGRPO: Flow's drift with a constant diffusion coefficient ``std = η``."""

    canonical_name: ClassVar[str] = "dance"

    def __init__(self, *, config: Optional["DanceSpec"] = None) -> None:
        pass

    def coeffs(self, sigma, sigma_next, eta, sigma_max):
        dt = sigma_next - sigma
        std = torch.full_like(sigma, eta)
        a_x, a_v = _flow_mean_coeffs(std, sigma, dt)
        return TransitionCoeffs(a_x, a_v, std * torch.sqrt(-dt))


class CPSSDEStrategy(SDEStrategy):
    """Coefficient-preserving sampling: ``std = σ'·sin(ηπ/2)``; ``mean = x̂0(1−σ') + ε̂·sqrt(σ'² − std²)``."""

    canonical_name: ClassVar[str] = "cps"

    def __init__(self, *, config: Optional["CPSSpec"] = None) -> None:
        pass

    def coeffs(self, sigma, sigma_next, eta, sigma_max):
        std = sigma_next * math.sin(eta * math.pi / 2)
        keep = torch.sqrt(sigma_next**2 - std**2)
        # x̂0 = x − σ v ; ε̂ = x + (1−σ) v
        a_x = (1 - sigma_next) + keep
        a_v = -(1 - sigma_next) * sigma + keep * (1 - sigma)
        return TransitionCoeffs(a_x, a_v, std, LOGP_NEG_SQ)


class DPM2Strategy(StepStrategy):
    """Second-order multistep DPM-Solver on the flow parameterisation (``α = 1−σ``); deterministic, stateful."""

    canonical_name: ClassVar[str] = "dpm2"

    def __init__(self, *, config: Optional["DPM2Spec"] = None) -> None:
        self.reset()

    def reset(self) -> None:
        self._sigmas: Optional[torch.Tensor] = None
        self._x0_hist: List[torch.Tensor] = []
        self._warm = 0

    def init_schedule(self, sigmas: torch.Tensor) -> None:
        self.reset()
        self._sigmas = sigmas

    @staticmethod
    def _lam(sig: torch.Tensor) -> torch.Tensor:
        return torch.log(1 - sig) - torch.log(sig)

    def denoise(self, noise_pred, sample, sigma, sigma_next, *, eta=1.0, prev_sample=None, sigma_max=0.99, step_index=0,
                noise=None, generator=None):
        if self._sigmas is None:
            raise RuntimeError("DPM2Strategy needs init_schedule() before stepping")
        v, x = noise_pred.float(), sample.float()
        sig = self._sigmas.to(x.device)
        n_steps = sig.numel() - 1
        x0 = x - sig[step_index].float() * v
        self._x0_hist = (self._x0_hist + [x0])[-2:]
        last = step_index == n_steps - 1
        second_to_last_short = step_index == n_steps - 2 and n_steps < 15
        s64 = sig.double()
        if self._warm < 1 or last:
            if step_index == 0 or last:
                t, s = sig[step_index + 1].float(), sig[step_index].float()
                eps = (x - (1 - s) * x0) / s
                out = (1 - t) * x0 + t.abs() * eps
            else:
                out = self._first_order(x0, s64, step_index, x)
        elif self._warm >= 1 or second_to_last_short:
            out = self._second_order(s64, step_index, x)
        self._warm = min(self._warm + 1, 2)
        return out.to(v.dtype), None, None

    def _first_order(self, x0, s, i, x):
        h = self._lam(s[i + 1]) - self._lam(s[i])
        return (s[i + 1] / s[i]) * x - ((1 - s[i + 1]) * (torch.exp(-h) - 1.0)) * x0

    def _second_order(self, s, i, x):
        m0, m1 = self._x0_hist[-1], self._x0_hist[-2]
        lam_t, lam_0, lam_1 = self._lam(s[i + 1]), self._lam(s[i]), self._lam(s[i - 1])
        h, h0 = lam_t - lam_0, lam_0 - lam_1
        d1 = (h / h0) * (m0 - m1)
        k = (1 - s[i + 1]) * (torch.exp(-h) - 1.0)
        return (s[i + 1] / s[i]) * x - k * m0 - 0.5 * k * d1


@dataclass
class FlowSpec:
    """FlowSDEStrategy has no per-instance settings."""


@dataclass
class CPSSpec:
    """CPSSDEStrategy has no per-instance settings."""


@dataclass
class DanceSpec:
    """DanceSDEStrategy has no per-instance settings."""


@dataclass
class DPM2Spec:
    """DPM2Strategy has no per-instance settings."""


STRATEGIES = {"flow": FlowSDEStrategy, "sde": FlowSDEStrategy, "cps": CPSSDEStrategy, "dance": DanceSDEStrategy,
              "dpm2": DPM2Strategy, "ode": StepStrategy}


def make_strategy(name: str) -> StepStrategy:
    try:
        return STRATEGIES[str(name).lower()]()
    except KeyError:
        raise ValueError(f"unknown SDE strategy '{name}' (have {sorted(STRATEGIES)})") from None


__all__ = ["StepStrategy", "SDEStrategy", "FlowSDEStrategy", "CPSSDEStrategy", "DanceSDEStrategy", "DPM2Strategy",
           "FlowSpec", "CPSSpec", "DanceSpec", "DPM2Spec", "TransitionCoeffs", "make_strategy", "LOGP_GAUSSIAN", "LOGP_NEG_SQ"]
