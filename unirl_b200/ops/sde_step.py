"""Fused SDE transition (K8): ``(v, x, coefficients, ε | x')`` → ``x'``, ``mean``, per-sample mean log-prob.

One pass over the latent replaces the ~12 element-wise launches of an eager implementation: the
kernel forms ``mean = a_x·x + a_v·v``, adds ``s·ε`` (sampling) or takes the stored ``x'`` (replay),
round-trips ``x'`` through the storage dtype, evaluates the log-prob element-wise and block-reduces
it to one value per sample.  Optional classifier-free-guidance combine (``v = v_u + g·(v_c − v_u)``) is
folded in.  Training replay stays differentiable through ``mean`` via a custom autograd node whose
backward is one kernel as well.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native
from unirl_b200.sde.kernels import LOGP_GAUSSIAN, LOGP_NEG_SQ, SDEStrategy, StepStrategy, _expand

import math

_HALF_LOG_2PI = 0.5 * math.log(2 * math.pi)


class _FusedReplay(torch.autograd.Function):
    """Replay-mode transition: differentiable w.r.t. the model output ``v``."""

    @staticmethod
    def forward(ctx, v, x, prev, a_x, a_v, std, logp_mode: int, v_uncond=None, guidance: float = 1.0):
        C = require_ext()
        vu = None if v_uncond is None else v_uncond.contiguous()
        mean, logp = C.sde_replay_fwd(v.contiguous(), x.contiguous(), prev.contiguous(), a_x, a_v, std, int(logp_mode), vu, float(guidance))
        count_launch()
        ctx.save_for_backward(mean, prev, a_v, std)
        ctx.mode, ctx.vdtype, ctx.guided, ctx.guidance = int(logp_mode), v.dtype, v_uncond is not None, float(guidance)
        return mean, logp

    @staticmethod
    def backward(ctx, g_mean, g_logp):
        C = require_ext()
        mean, prev, a_v, std = ctx.saved_tensors
        gm = g_mean.contiguous() if g_mean is not None else None
        gv = C.sde_replay_bwd(gm, g_logp.float().contiguous(), mean, prev, a_v, std, ctx.mode, ctx.guided, ctx.guidance)
        count_launch()
        if ctx.guided:
            return gv[0].to(ctx.vdtype), None, None, None, None, None, None, gv[1].to(ctx.vdtype), None
        return gv.to(ctx.vdtype), None, None, None, None, None, None, None, None


def sde_step(strategy: StepStrategy, noise_pred: torch.Tensor, sample: torch.Tensor, sigma: torch.Tensor, sigma_next: torch.Tensor, *,
             eta: float = 1.0, prev_sample: Optional[torch.Tensor] = None, sigma_max: float = 0.99, step_index: int = 0,
             noise: Optional[torch.Tensor] = None, generator: Optional[torch.Generator] = None,
             noise_pred_uncond: Optional[torch.Tensor] = None, guidance_scale: float = 1.0,
             ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Drop-in for ``strategy.denoise`` that uses the fused kernel for stochastic strategies on CUDA.

    With ``noise_pred_uncond`` the two branches of a classifier-free-guidance pass are combined inside the kernel
    (``v = v_u + g·(v_c − v_u)`` with ``noise_pred`` as ``v_c``), forward and backward; elsewhere the combination is formed first."""
    if not (use_native(noise_pred) and isinstance(strategy, SDEStrategy) and eta >= 1e-7):
        if noise_pred_uncond is not None:
            noise_pred = noise_pred_uncond + guidance_scale * (noise_pred - noise_pred_uncond)
        return strategy.denoise(noise_pred, sample, sigma, sigma_next, eta=eta, prev_sample=prev_sample, sigma_max=sigma_max,
                                step_index=step_index, noise=noise, generator=generator)
    b = sample.shape[0]
    c = strategy.coeffs(_expand(sigma, 1), _expand(sigma_next, 1), float(eta), float(sigma_max))
    per_sample = lambda t: t.reshape(-1).float().expand(b).contiguous()  # noqa: E731
    a_x, a_v, std = per_sample(c.a_x), per_sample(c.a_v), per_sample(c.noise_std)
    if prev_sample is not None:
        prev = prev_sample.to(sample.dtype)
        mean, logp = _FusedReplay.apply(noise_pred, sample, prev, a_x, a_v, std, c.logp_mode, noise_pred_uncond, float(guidance_scale))
        return prev.float(), logp, mean
    C = require_ext()
    if noise is None:
        noise = torch.randn(noise_pred.shape, dtype=torch.float32, device=noise_pred.device, generator=generator)
    prev, mean, logp = C.sde_sample_fwd(noise_pred.contiguous(), sample.contiguous(), noise.contiguous(), a_x, a_v, std, int(c.logp_mode),
                                        None if noise_pred_uncond is None else noise_pred_uncond.contiguous(), float(guidance_scale))
    count_launch()
    return prev, logp, mean


__all__ = ["sde_step"]
