"""Fused AdamW (K10) over a flat fp32 master shard.

The sharded trainer keeps, per parameter group, ONE flat fp32 master buffer, flat ``exp_avg`` /
``exp_avg_sq`` and a flat bf16 compute copy.  A step is a single kernel over the flat shard:
unscale/clip the gradient, update both moments, apply decoupled weight decay, write the fp32
master and the bf16 copy, and (optionally) lerp an EMA shadow — instead of the reference's
per-tensor ``torch.optim.AdamW(foreach=False)`` launches (``unirl/train/factories.py:51-58``) plus a
separate EMA loop (``unirl/train/ema.py:52-60``).
"""

from __future__ import annotations

from typing import Optional

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native


def adamw_reference(master: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, *, lr: float,
                    beta1: float, beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
                    low: Optional[torch.Tensor] = None, ema: Optional[torch.Tensor] = None, ema_decay: float = 0.0) -> None:
    g = grad.float() * grad_scale
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1**step, 1 - beta2**step
    master.mul_(1 - lr * weight_decay)
    master.addcdiv_(exp_avg, (exp_avg_sq / bc2).sqrt_().add_(eps), value=-lr / bc1)
    if low is not None:
        low.copy_(master)
    if ema is not None:
        ema.mul_(ema_decay).add_(master, alpha=1 - ema_decay)


def adamw_step(master: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, *, lr: float,
               beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0, step: int = 1,
               grad_scale: float = 1.0, low: Optional[torch.Tensor] = None, ema: Optional[torch.Tensor] = None,
               ema_decay: float = 0.0, grad_scale_tensor: Optional[torch.Tensor] = None) -> None:
    """In-place AdamW on flat buffers; ``grad`` may be bf16 or fp32.  ``grad_scale_tensor`` (device
    fp32 scalar, multiplied with ``grad_scale``) carries the clip coefficient without a host sync."""
    if use_native(master):
        require_ext().adamw_step(master, grad, exp_avg, exp_avg_sq, low, ema, float(lr), float(beta1), float(beta2), float(eps),
                                 float(weight_decay), int(step), float(grad_scale), float(ema_decay), grad_scale_tensor)
        count_launch()
        return
    if grad_scale_tensor is not None:
        grad_scale = grad_scale * float(grad_scale_tensor)
    adamw_reference(master, grad, exp_avg, exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
                    grad_scale=grad_scale, low=low, ema=ema, ema_decay=ema_decay)


def sum_squares(x: torch.Tensor) -> torch.Tensor:
    """fp32 Σx² of a flat buffer (partial of the global grad norm)."""
    if use_native(x):
        out = require_ext().sum_squares(x)
        count_launch()
        return out
    return x.float().pow(2).sum()


__all__ = ["adamw_step", "adamw_reference", "sum_squares"]
