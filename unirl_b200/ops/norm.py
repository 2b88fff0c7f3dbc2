"""RMSNorm family (K4): plain, fused residual-add, and adaLN modulate.

CUDA: one pass per row, fp32 accumulation, bf16 I/O, custom autograd with a fused backward kernel.
CPU / oracle: the fp32 PyTorch expression below.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native


def rmsnorm_reference(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        C = require_ext()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, rstd = C.rmsnorm_fwd(x2, weight, float(eps))
        count_launch()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, gy):
        C = require_ext()
        x2, weight, rstd = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1]).contiguous()
        gx, gw = C.rmsnorm_bwd(g2, x2, weight, rstd)
        count_launch()
        return gx.view(ctx.shape), gw.to(weight.dtype), None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x · rsqrt(mean(x²) + eps) · weight`` over the last dim."""
    if use_native(x):
        return _RMSNorm.apply(x, weight, eps)
    return rmsnorm_reference(x, weight, eps)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """``r' = residual + x``; returns ``(rmsnorm(r'), r')`` — inference path fuses both into one pass."""
    if use_native(x) and not torch.is_grad_enabled():
        C = require_ext()
        y, r = C.add_rmsnorm_fwd(x.contiguous(), residual.contiguous(), weight, float(eps))
        count_launch()
        return y, r
    r = residual + x
    return rmsnorm(r, weight, eps), r


def layernorm_modulate_reference(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    """adaLN: ``LayerNorm(x) · (1 + scale) + shift`` without affine params; shift/scale are ``[B, D]`` for ``x [B, L, D]``."""
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps)
    return (y * (1 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)).to(x.dtype)


class _LayerNormModulate(torch.autograd.Function):
    """adaLN forward and backward as one kernel each; the statistics are recomputed in the backward (nothing saved but the inputs)."""

    @staticmethod
    def forward(ctx, x, shift, scale, eps: float):
        x, shift, scale = x.contiguous(), shift.contiguous(), scale.contiguous()
        out = require_ext().layernorm_modulate_fwd(x, shift, scale, float(eps))
        count_launch()
        ctx.save_for_backward(x, scale)
        ctx.eps, ctx.mod_dtype = float(eps), shift.dtype
        return out

    @staticmethod
    def backward(ctx, gy):
        x, scale = ctx.saved_tensors
        dx, dshift, dscale = require_ext().layernorm_modulate_bwd(gy.contiguous(), x, scale, ctx.eps)
        count_launch()
        return dx, dshift.to(ctx.mod_dtype), dscale.to(ctx.mod_dtype), None


def layernorm_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if use_native(x) and x.dim() == 3 and shift.dtype == x.dtype and scale.dtype == x.dtype:
        if not (torch.is_grad_enabled() and (x.requires_grad or shift.requires_grad or scale.requires_grad)):
            out = require_ext().layernorm_modulate_fwd(x.contiguous(), shift.contiguous(), scale.contiguous(), float(eps))
            count_launch()
            return out
        if x.shape[-1] <= 6144:
            return _LayerNormModulate.apply(x, shift, scale, eps)
    return layernorm_modulate_reference(x, shift, scale, eps)


__all__ = ["rmsnorm", "add_rmsnorm", "layernorm_modulate", "rmsnorm_reference", "layernorm_modulate_reference"]
