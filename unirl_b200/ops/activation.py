"""SwiGLU on a fused ``[T, 2·I]`` gate|up projection: ``silu(gate) · up`` (fwd + bwd kernels)."""

from __future__ import annotations

import torch
import torch.nn.functional as F

from unirl_b200.ops._ext import count_launch, require_ext, use_native


def swiglu_reference(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, -1)
    return (F.silu(g) * u).to(gate_up.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        C = require_ext()
        gate_up = gate_up.contiguous()
        ctx.save_for_backward(gate_up)
        out = C.swiglu_fwd(gate_up)
        count_launch()
        return out

    @staticmethod
    def backward(ctx, gy):
        C = require_ext()
        (gate_up,) = ctx.saved_tensors
        out = C.swiglu_bwd(gy.contiguous(), gate_up)
        count_launch()
        return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    return _SwiGLU.apply(gate_up) if use_native(gate_up) else swiglu_reference(gate_up)


__all__ = ["swiglu", "swiglu_reference"]
