"""Policy-ratio losses (K7): PPO clip, DRPO quadratic penalty, Flow-DPPO KL mask.

Each function returns ``(loss_per_element, metrics)`` where metrics are detached 0-dim tensors.
On CUDA one fused kernel per family computes the loss, its derivative w.r.t. ``new_logp`` and the
metric reductions in a single pass (the derivative is replayed by a custom autograd node); on CPU
the same math is a PyTorch fp32 expression, which is also the test oracle.

Math parity: ``unirl/algorithms/base.py:115-157`` (clip), ``drpo.py:131-159``, ``flowdppo.py:54-138``.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native

Metrics = Dict[str, torch.Tensor]


# ------------------------------------------------------------------------------------- references
def ppo_clip_reference(new_logp, old_logp, adv, eps_lo: float, eps_hi: float) -> Tuple[torch.Tensor, Metrics]:
    log_diff = new_logp - old_logp
    ratio = torch.exp(log_diff)
    a = adv.detach()
    loss = torch.maximum(-a * ratio, -a * torch.clamp(ratio, 1.0 - eps_lo, 1.0 + eps_hi))
    with torch.no_grad():
        gt, lt = (ratio - 1.0 > eps_hi).float(), (1.0 - ratio > eps_lo).float()
        m = {"ratio_mean": ratio.mean(), "ratio_std": ratio.std() if ratio.numel() > 1 else ratio.new_zeros(()),
             "ratio_min": ratio.min(), "ratio_max": ratio.max(), "clip_fraction": torch.maximum(gt, lt).mean(),
             "clipfrac_gt_one": gt.mean(), "clipfrac_lt_one": lt.mean(), "approx_kl": (0.5 * log_diff.pow(2)).mean()}
    return loss, m


def drpo_reference(new_logp, old_logp, adv, epsilon: float, mu_weighted: bool) -> Tuple[torch.Tensor, Metrics]:
    log_diff = torch.clamp(new_logp - old_logp, -20.0, 20.0)
    ratio = torch.exp(log_diff)
    a = adv.detach()
    mu = torch.exp(old_logp).detach()
    if mu_weighted:
        w = mu
        eps_t = torch.where(mu > 0, epsilon / mu, torch.full_like(mu, float("inf")))
    else:
        w, eps_t = torch.ones_like(mu), torch.full_like(mu, epsilon)
    penalty = a.abs() * w * (ratio - 1.0).square() / (2.0 * epsilon)
    loss = -a * ratio + penalty
    with torch.no_grad():
        m = {"ratio_mean": ratio.mean(), "ratio_max": ratio.max(), "approx_kl": ((ratio - 1.0) - log_diff).mean(),
             "drpo_penalty_mean": penalty.mean(), "clipfrac_upper": (ratio > 1.0 + eps_t).float().mean(),
             "clipfrac_lower": (ratio < 1.0 - eps_t).float().mean()}
    return loss, m


def flow_dppo_reference(new_logp, old_logp, new_means, old_means, adv, sigma_t, tau: float) -> Tuple[torch.Tensor, Metrics]:
    log_diff = new_logp - old_logp
    ratio = torch.exp(log_diff)
    a = adv.detach()
    kl = ((new_means - old_means) ** 2 / (2 * sigma_t**2)).mean(dim=tuple(range(2, new_means.dim())))
    low_kl = kl < tau
    pos = (~low_kl) & (ratio > 1.0) & (a > 0)
    neg = (~low_kl) & (ratio < 1.0) & (a < 0)
    keep = (~(pos | neg)).detach()
    loss = torch.where(keep, -a * ratio, ratio.new_zeros(()))
    with torch.no_grad():
        m = {"ratio_mean": ratio.mean(), "ratio_std": ratio.std() if ratio.numel() > 1 else ratio.new_zeros(()),
             "ratio_min": ratio.min(), "ratio_max": ratio.max(), "approx_kl": (0.5 * log_diff.pow(2)).mean(),
             "kl_new_old_mean": kl.mean(), "kl_new_old_max": kl.max(), "kl_mask_fraction": (~low_kl).float().mean(),
             "pos_rm_fraction": pos.float().mean(), "neg_rm_fraction": neg.float().mean(),
             "masked_fraction": (pos | neg).float().mean(), "unmasked_fraction": keep.float().mean()}
    return loss, m


# ------------------------------------------------------------------------------------- fused path
class _FusedElementwiseLoss(torch.autograd.Function):
    """loss_i = f(new_i; old_i, adv_i, params); the kernel also emits f'(new_i) for backward."""

    @staticmethod
    def forward(ctx, new_logp, old_logp, adv, kind: int, p0: float, p1: float, keep_mask):
        C = require_ext()
        shape = new_logp.shape
        n = new_logp.reshape(-1).float().contiguous()
        o = old_logp.reshape(-1).float().contiguous()
        a = adv.reshape(-1).float().contiguous()
        k = keep_mask.reshape(-1).to(torch.uint8).contiguous() if keep_mask is not None else None
        loss, dloss, stats = C.policy_loss_fwd(n, o, a, k, int(kind), float(p0), float(p1))
        count_launch()
        ctx.save_for_backward(dloss)
        ctx.shape = shape
        ctx.mark_non_differentiable(stats)
        return loss.view(shape), stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        (dloss,) = ctx.saved_tensors
        return (g_loss.reshape(-1) * dloss).view(ctx.shape).to(g_loss.dtype), None, None, None, None, None, None


_KIND_CLIP, _KIND_DRPO, _KIND_DRPO_PLAIN, _KIND_MASKED_PG = 0, 1, 2, 3


def _stats_common(stats: torch.Tensor, n: int) -> Metrics:
    # stats layout: [sum_r, sum_r2, min_r, max_r, sum_a, sum_b, sum_c, sum_kl]
    mean = stats[0] / n
    var = (stats[1] / n - mean * mean).clamp(min=0) * (n / max(n - 1, 1))
    return {"ratio_mean": mean, "ratio_std": var.sqrt() if n > 1 else mean.new_zeros(()), "ratio_min": stats[2], "ratio_max": stats[3]}


def ppo_clip(new_logp, old_logp, adv, eps_lo: float, eps_hi: float) -> Tuple[torch.Tensor, Metrics]:
    if not use_native(new_logp):
        return ppo_clip_reference(new_logp, old_logp, adv, eps_lo, eps_hi)
    loss, s = _FusedElementwiseLoss.apply(new_logp, old_logp, adv, _KIND_CLIP, eps_lo, eps_hi, None)
    n = new_logp.numel()
    m = _stats_common(s, n)
    m.update({"clip_fraction": (s[4] + s[5]) / n, "clipfrac_gt_one": s[4] / n, "clipfrac_lt_one": s[5] / n, "approx_kl": s[7] / n})
    return loss, m


def drpo(new_logp, old_logp, adv, epsilon: float, mu_weighted: bool) -> Tuple[torch.Tensor, Metrics]:
    if not use_native(new_logp):
        return drpo_reference(new_logp, old_logp, adv, epsilon, mu_weighted)
    loss, s = _FusedElementwiseLoss.apply(new_logp, old_logp, adv, _KIND_DRPO if mu_weighted else _KIND_DRPO_PLAIN, epsilon, 0.0, None)
    n = new_logp.numel()
    return loss, {"ratio_mean": s[0] / n, "ratio_max": s[3], "approx_kl": s[7] / n, "drpo_penalty_mean": s[6] / n,
                  "clipfrac_upper": s[4] / n, "clipfrac_lower": s[5] / n}


def flow_dppo(new_logp, old_logp, new_means, old_means, adv, sigma_t, tau: float) -> Tuple[torch.Tensor, Metrics]:
    if not use_native(new_logp):
        return flow_dppo_reference(new_logp, old_logp, new_means, old_means, adv, sigma_t, tau)
    C = require_ext()
    b, s_ = new_logp.shape
    inv2s2 = (1.0 / (2 * sigma_t.float() ** 2)).reshape(-1)
    inv2s2 = inv2s2.expand(s_).contiguous() if inv2s2.numel() == 1 else inv2s2.contiguous()
    with torch.no_grad():
        kl = C.mean_sq_diff_rows(new_means.detach().reshape(b * s_, -1).contiguous(), old_means.reshape(b * s_, -1).contiguous()).view(b, s_) * inv2s2.view(1, s_)
        count_launch()
        ratio_dir = torch.exp(new_logp.detach() - old_logp)
        a = adv.detach()
        low_kl = kl < tau
        pos = (~low_kl) & (ratio_dir > 1.0) & (a > 0)
        neg = (~low_kl) & (ratio_dir < 1.0) & (a < 0)
        keep = ~(pos | neg)
    loss, st = _FusedElementwiseLoss.apply(new_logp, old_logp, adv, _KIND_MASKED_PG, 0.0, 0.0, keep)
    n = new_logp.numel()
    m = _stats_common(st, n)
    m.update({"approx_kl": st[7] / n, "kl_new_old_mean": kl.mean(), "kl_new_old_max": kl.max(),
              "kl_mask_fraction": (~low_kl).float().mean(), "pos_rm_fraction": pos.float().mean(), "neg_rm_fraction": neg.float().mean(),
              "masked_fraction": (pos | neg).float().mean(), "unmasked_fraction": keep.float().mean()})
    return loss, m


__all__ = ["ppo_clip", "drpo", "flow_dppo", "ppo_clip_reference", "drpo_reference", "flow_dppo_reference"]
