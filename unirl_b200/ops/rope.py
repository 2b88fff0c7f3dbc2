"""Rotary position embedding fused with per-head q/k RMSNorm (K4+K5), applied to packed QKV.

``qkv`` is ``[T, (Hq + 2·Hkv)·D]`` straight out of the fused QKV GEMM.  The op normalises every q
and k head (Qwen3 QK-norm; pass ``None`` weights to skip), rotates them by ``positions`` with the
half-split ("NeoX") convention and leaves v untouched.  The backward kernel undoes the rotation and
the norm in one pass.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from unirl_b200.ops._ext import count_launch, require_ext, use_native


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float().unsqueeze(-1) * inv
    return ang.cos(), ang.sin()


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def qk_norm_rope_reference(qkv, q_weight, k_weight, positions, n_q, n_kv, head_dim, theta, eps):
    t = qkv.shape[0]
    q, k, v = qkv.float().split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], -1)
    q, k = q.view(t, n_q, head_dim), k.view(t, n_kv, head_dim)
    if q_weight is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight.float()
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight.float()
    cos, sin = rope_cos_sin(positions, head_dim, theta)
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
    return q.to(qkv.dtype), k.to(qkv.dtype), v.reshape(t, n_kv, head_dim).to(qkv.dtype)


class _QKNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, positions, n_q, n_kv, head_dim, theta, eps):
        C = require_ext()
        qkv = qkv.contiguous()
        q, k, v, rstd = C.qk_norm_rope_fwd(qkv, q_weight, k_weight, positions.to(torch.int32), n_q, n_kv, head_dim, float(theta), float(eps))
        count_launch()
        ctx.save_for_backward(qkv, q_weight, k_weight, positions, rstd)
        ctx.cfg = (n_q, n_kv, head_dim, float(theta), float(eps))
        return q, k, v

    @staticmethod
    def backward(ctx, gq, gk, gv):
        C = require_ext()
        qkv, qw, kw, positions, rstd = ctx.saved_tensors
        n_q, n_kv, head_dim, theta, eps = ctx.cfg
        g_qkv, g_qw, g_kw = C.qk_norm_rope_bwd(gq.contiguous(), gk.contiguous(), gv.contiguous(), qkv, qw, kw,
                                               positions.to(torch.int32), rstd, n_q, n_kv, head_dim, theta)
        count_launch()
        return g_qkv, (g_qw.to(qw.dtype) if qw is not None else None), (g_kw.to(kw.dtype) if kw is not None else None), None, None, None, None, None, None


def qk_norm_rope(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], positions: torch.Tensor,
                 n_q: int, n_kv: int, head_dim: int, theta: float = 1e6, eps: float = 1e-6):
    """Returns ``q [T,Hq,D]``, ``k [T,Hkv,D]``, ``v [T,Hkv,D]``."""
    if use_native(qkv) and q_weight is not None:
        return _QKNormRope.apply(qkv, q_weight, k_weight, positions, n_q, n_kv, head_dim, theta, eps)
    return qk_norm_rope_reference(qkv, q_weight, k_weight, positions, n_q, n_kv, head_dim, theta, eps)


def qk_norm_rope_cached(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], positions: torch.Tensor, n_q: int, n_kv: int,
                        head_dim: int, theta: float, eps: float, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor, dense_kv: bool):
    """Inference: QK-norm + rotary + KV-cache write.  Returns ``(q, k | None, v | None)``; ``dense_kv=False`` (decode) skips the
    ``[T, Hkv, D]`` copies because attention reads the cache.  One launch on CUDA (bf16, head_dim 128 / 256, QK-norm on)."""
    if use_native(qkv) and q_weight is not None and qkv.dtype == torch.bfloat16 and head_dim in (128, 256) and not torch.is_grad_enabled():
        out = require_ext().qk_norm_rope_cache_fwd(qkv.contiguous(), q_weight, k_weight, positions.to(torch.int32), k_cache, v_cache, slot_mapping, n_q, n_kv,
                                                   head_dim, float(theta), float(eps), bool(dense_kv))
        count_launch()
        return (out[0], out[1], out[2]) if dense_kv else (out[0], None, None)
    from unirl_b200.ops.attention import kv_cache_write

    q, k, v = qk_norm_rope(qkv, q_weight, k_weight, positions, n_q, n_kv, head_dim, theta, eps)
    kv_cache_write(k, v, k_cache, v_cache, slot_mapping)
    return q, k, v


class _RopeTable(torch.autograd.Function):
    """Rotation by per-token tables; the gradient is the rotation by the opposite angle."""

    @staticmethod
    def forward(ctx, x, cos, sin, interleaved: bool):
        y = require_ext().rope_table(x.contiguous(), cos, sin, bool(interleaved), False)
        count_launch()
        ctx.save_for_backward(cos, sin)
        ctx.interleaved = bool(interleaved)
        return y

    @staticmethod
    def backward(ctx, gy):
        cos, sin = ctx.saved_tensors
        gx = require_ext().rope_table(gy.contiguous(), cos, sin, ctx.interleaved, True)
        count_launch()
        return gx, None, None, None


def rope_table_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """fp32 statement of the table-driven rotation: ``x [..., L, H, D]``, ``cos / sin [L, D/2]``."""
    xf = x.float()
    c, s = cos.float().unsqueeze(-2), sin.float().unsqueeze(-2)  # [L, 1, D/2]
    if interleaved:
        p = xf.unflatten(-1, (-1, 2))
        a, b = p[..., 0], p[..., 1]
        return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2).to(x.dtype)
    h = x.shape[-1] // 2
    a, b = xf[..., :h], xf[..., h:]
    return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)


def rope_table(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """Rotate ``x [..., L, H, D]`` by per-token angle tables ``cos / sin [L, D/2]`` (any leading batch dimensions share the tables).
    ``interleaved``: pairs ``(2i, 2i+1)`` (axial 3-D rotary of the diffusion transformers); otherwise ``(i, i + D/2)`` (3-axis rotary of
    the vision-language decoder).  One kernel forward, one backward."""
    if use_native(x) and x.dtype in (torch.bfloat16, torch.float32):
        return _RopeTable.apply(x, cos.float().contiguous(), sin.float().contiguous(), bool(interleaved))
    return rope_table_reference(x, cos, sin, interleaved)


def mrope_cos_sin(positions3: torch.Tensor, head_dim: int, theta: float, sections: Tuple[int, int, int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Multimodal rotary tables: frequency ``j`` takes its position from the temporal, height or width axis according to
    ``sections`` (counts of frequencies per axis, summing to ``head_dim / 2``).  ``positions3`` is ``[3, T]``."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions3.device, dtype=torch.float32) / head_dim))
    axis = torch.repeat_interleave(torch.arange(3, device=positions3.device), torch.tensor(list(sections), device=positions3.device))
    pos = positions3.float()[axis].transpose(0, 1)  # [T, D/2]: the position each frequency sees
    ang = pos * inv
    return ang.cos(), ang.sin()


def mrope_qk(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], positions3: torch.Tensor, n_q: int, n_kv: int,
             head_dim: int, theta: float, eps: float, sections: Tuple[int, int, int]):
    """QK-norm + 3-axis rotary for vision-language prompts (prefill / training; decode positions collapse to one axis
    and take the fused kernel).  On CUDA: the per-head RMS-norm kernel, then the table-driven rotary kernel (both differentiable);
    elsewhere the PyTorch composition below."""
    t = qkv.shape[0]
    if use_native(qkv) and qkv.dtype in (torch.bfloat16, torch.float32):
        from unirl_b200.ops.norm import rmsnorm

        q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], -1)
        q, k = q.reshape(t, n_q, head_dim), k.reshape(t, n_kv, head_dim)
        if q_weight is not None:
            q = rmsnorm(q.reshape(-1, head_dim), q_weight, eps).view(t, n_q, head_dim)
            k = rmsnorm(k.reshape(-1, head_dim), k_weight, eps).view(t, n_kv, head_dim)
        cos, sin = mrope_cos_sin(positions3, head_dim, theta, sections)
        return rope_table(q, cos, sin, False), rope_table(k, cos, sin, False), v.reshape(t, n_kv, head_dim).contiguous()
    q, k, v = qkv.float().split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], -1)
    q, k = q.view(t, n_q, head_dim), k.view(t, n_kv, head_dim)
    if q_weight is not None:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight.float()
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight.float()
    cos, sin = mrope_cos_sin(positions3, head_dim, theta, sections)
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return _rotate(q, cos, sin).to(qkv.dtype), _rotate(k, cos, sin).to(qkv.dtype), v.reshape(t, n_kv, head_dim).to(qkv.dtype)


__all__ = ["qk_norm_rope", "qk_norm_rope_reference", "qk_norm_rope_cached", "rope_cos_sin", "mrope_qk", "mrope_cos_sin", "rope_table", "rope_table_reference"]
