"""Linear layers (K1): ``y = x · Wᵀ`` with optional fused epilogues.

Forward and backward on CUDA go to the hand-written tcgen05/TMEM GEMM (TMA-fed, persistent, 128×256 tiles).  The kernel
takes each operand K-major or MN-major, so ``dX = dY·W`` reads ``W`` as stored and ``dW = dYᵀ·X`` reads ``dY`` and ``X``
as stored (no transpose pass); the weight gradient accumulates in fp32 straight into the trainer's buffer from the
epilogue.  ``UNIRL_B200_GEMM_BWD=library`` restores library GEMMs in backward (A/B measurements).
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F

from unirl_b200.ops._ext import count_launch, ext, require_ext, use_native

# The persistent 128x256-tile tcgen05 kernel takes the compute-bound shapes (prefill, training forward) where whole tiles
# fill the machine.  Decode-shaped GEMMs (M up to _MAX_SKINNY_M rows, no autograd) are weight-bandwidth bound and go to the
# cluster split-K kernel: one tile per CTA, the K range split over a thread-block cluster and summed through distributed shared memory.
_MIN_NATIVE_M = int(os.environ.get("UNIRL_B200_GEMM_MIN_M", "512"))
_WGRAD_FUSION = os.environ.get("UNIRL_B200_WGRAD_FUSION", "1") != "0"
_MAX_SKINNY_M = int(os.environ.get("UNIRL_B200_GEMM_SKINNY_MAX_M", "128"))  # measured win at one 128-row tile; 256 rows (two tiles re-reading the weights) lose to the library
# "unsplit": only shapes whose tiles fill a wave without splitting K (the cluster exchange costs about what the library's
# split-K costs, so those shapes stay on the library GEMM); "all": every qualifying shape.
_SKINNY_MODE = os.environ.get("UNIRL_B200_GEMM_SKINNY_MODE", "unsplit")
_BWD_NATIVE = os.environ.get("UNIRL_B200_GEMM_BWD", "native") == "native"
_plan_cache: dict = {}


def _bwd_native_ok(g2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor) -> bool:
    return (_BWD_NATIVE and g2.dtype == torch.bfloat16 and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and g2.shape[0] >= _MIN_NATIVE_M
            and g2.shape[1] % 8 == 0 and x2.shape[1] % 8 == 0 and g2.stride(1) == 1 and g2.stride(0) % 8 == 0
            and hasattr(ext(), "gemm_bf16"))


def _skinny_unsplit(m: int, n: int, k: int, swiglu: bool) -> bool:
    key = (m, n, k, swiglu)
    if key not in _plan_cache:
        _plan_cache[key] = int(ext().gemm_skinny_plan(m, n, k, swiglu)[1]) == 1
    return _plan_cache[key]


def _skinny_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    m, k = x2.shape
    n = w.shape[0]
    return (0 < m <= _MAX_SKINNY_M and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 64 == 0 and n % 8 == 0 and n >= 1024
            and w.is_contiguous() and os.environ.get("UNIRL_B200_GEMM", "native") == "native")


def skinny_linear(x2: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  epilogue: int = 0) -> Optional[torch.Tensor]:
    """Inference-only ``x2 @ weightᵀ (+ residual)`` -- or, with ``epilogue=EPI_SWIGLU`` and ``weight = [Wg; Wu]``,
    ``silu(x2·Wgᵀ) ⊙ (x2·Wuᵀ)`` -- for a decode-sized ``x2 [M, K]`` through the cluster split-K tcgen05 GEMM;
    ``None`` when the shape does not qualify (the caller then uses the library GEMM)."""
    C = ext()
    if C is None or not hasattr(C, "gemm_bf16_tn_skinny") or not x2.is_cuda or not _skinny_ok(x2, weight):
        return None
    swiglu = int(epilogue) == EPI_SWIGLU
    if _SKINNY_MODE != "all" and not _skinny_unsplit(x2.shape[0], weight.shape[0] // (2 if swiglu else 1), x2.shape[1], swiglu):
        return None
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if residual is not None and not residual.is_contiguous():
        residual = residual.contiguous()
    y = C.gemm_bf16_tn_skinny(x2, weight, residual, out, int(epilogue))
    count_launch()
    return y


def _native_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    m, k = x2.shape
    n = w.shape[0]
    return (x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 64 == 0 and n % 16 == 0 and m >= _MIN_NATIVE_M
            and x2.is_contiguous() and w.is_contiguous() and os.environ.get("UNIRL_B200_GEMM", "native") == "native")


class _NativeLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, epilogue: int):
        C = require_ext()
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.reshape(-1, residual.shape[-1]).contiguous() if residual is not None else None
        y = C.gemm_bf16_tn(x2, w, res2, int(epilogue))
        count_launch()
        ctx.save_for_backward(x2, w)
        ctx.has_res = residual is not None
        ctx.in_shape = x.shape
        # set by the sharded trainer on its parameters: returns the fp32 gradient-accumulator view of this weight
        ctx.accum = getattr(w, "_wgrad_accum", None) if _WGRAD_FUSION else None
        ctx.param = w if ctx.accum is not None else None
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        g2 = gy.reshape(-1, gy.shape[-1])
        if _bwd_native_ok(g2, x2, w):
            C = require_ext()
            gx = gw = None
            if ctx.needs_input_grad[0]:
                gx = C.gemm_bf16(g2, w, False, True).view(ctx.in_shape)  # dX = dY·W, W read as stored ([N, K] = MN-major B)
                count_launch()
            if ctx.needs_input_grad[1]:
                if ctx.accum is not None:
                    # dW += dYᵀ·X with both operands read as stored; fp32 accumulation into the trainer's buffer happens in the epilogue,
                    # so neither a bf16 dW nor a separate add pass exists.  Autograd still needs a gradient object to fire the
                    # parameter's hook; an uninitialised placeholder costs nothing.
                    C.gemm_bf16(g2, x2, True, True, ctx.accum(), True)
                    ctx.param._wgrad_fused = True
                    gw = torch.empty(w.shape, dtype=w.dtype, device=w.device)
                else:
                    gw = C.gemm_bf16(g2, x2, True, True)
                count_launch()
            return gx, gw, (gy if ctx.has_res else None), None
        gx = (g2 @ w).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        gw = None
        if ctx.needs_input_grad[1]:
            if ctx.accum is not None:
                # dW accumulates into the fp32 buffer inside the GEMM (C = 1·C + dYᵀ·X, fp32 output): the bf16 dW and the
                # separate add pass (12 bytes of traffic per parameter and micro-batch) disappear.  Autograd still needs a
                # gradient object to fire the parameter's hook; an uninitialised placeholder costs nothing.
                acc = ctx.accum()
                torch.addmm(acc, g2.t(), x2, out_dtype=torch.float32, out=acc)
                ctx.param._wgrad_fused = True
                gw = torch.empty(w.shape, dtype=w.dtype, device=w.device)
            else:
                gw = g2.t() @ x2
        return gx, gw, (gy if ctx.has_res else None), None


def linear_grads(g2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, need_x: bool = True, need_w: bool = True):
    """``(dX, dW)`` of ``y = x2 · wᵀ`` for an upstream gradient ``g2 [M, N]``: the tcgen05 GEMM with the operands read as stored, the
    library for shapes it does not take.  For autograd functions that produce ``y`` in a form of their own."""
    if _bwd_native_ok(g2, x2, w):
        C = require_ext()
        gx = C.gemm_bf16(g2, w, False, True) if need_x else None
        gw = C.gemm_bf16(g2, x2, True, True) if need_w else None
        count_launch((1 if need_x else 0) + (1 if need_w else 0))
        return gx, gw
    return (g2 @ w if need_x else None), (g2.t() @ x2 if need_w else None)


EPI_NONE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2


def linear(x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weightᵀ (+ residual)``; ``weight`` is ``[out, in]``."""
    if use_native(x):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if ext() is not None and hasattr(ext(), "gemm_bf16_tn") and _native_ok(x2, weight):
            return _NativeLinear.apply(x, weight, residual, EPI_RESIDUAL if residual is not None else EPI_NONE)
        if not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or (residual is not None and residual.requires_grad))):
            y = skinny_linear(x2, weight, residual.reshape(-1, residual.shape[-1]) if residual is not None else None)
            if y is not None:
                return y.view(*x.shape[:-1], y.shape[-1])
    y = F.linear(x, weight)
    return y + residual if residual is not None else y


def linear_swiglu(x: torch.Tensor, weight_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x·Wgᵀ) · (x·Wuᵀ)`` with ``weight_gate_up = [Wg; Wu]`` (``[2I, in]``).

    Inference path fuses the activation into the GEMM epilogue (gate/up rows interleaved per tile by
    the weight packer); training keeps GEMM and activation as two autograd nodes.
    """
    from unirl_b200.ops.activation import swiglu

    if use_native(x) and not (torch.is_grad_enabled() and (x.requires_grad or weight_gate_up.requires_grad)) and weight_gate_up.shape[0] % 16 == 0:
        y = skinny_linear(x.reshape(-1, x.shape[-1]), weight_gate_up, epilogue=EPI_SWIGLU)
        if y is not None:
            return y.view(*x.shape[:-1], y.shape[-1])
    return swiglu(linear(x, weight_gate_up))


def lora_linear(x: torch.Tensor, weight: torch.Tensor, lora_a: torch.Tensor, lora_b: torch.Tensor, scaling: float,
                bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x·Wᵀ + scaling · (x·Aᵀ)·Bᵀ`` — the rank-r path is two skinny GEMMs accumulated onto the base output."""
    y = linear(x, weight)
    y = y + (F.linear(F.linear(x, lora_a), lora_b) * scaling).to(y.dtype)
    return y + bias if bias is not None else y


__all__ = ["linear", "skinny_linear", "linear_swiglu", "lora_linear", "EPI_NONE", "EPI_RESIDUAL", "EPI_SWIGLU"]
