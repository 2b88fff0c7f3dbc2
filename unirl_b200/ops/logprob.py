"""Token log-prob (K6): ``log softmax(h·Wᵀ / T)[target]`` without ever materialising ``[tokens, vocab]`` in fp32.

CUDA forward: the tcgen05 GEMM runs over vocab tiles with an epilogue that reduces each 128×N
accumulator tile (still in TMEM) to per-row ``(max, Σexp, target logit)`` partials; a merge kernel
folds the partials into ``lse`` and ``logp``.  Logits never reach HBM.
CUDA backward: per token chunk, the same GEMM recomputes the logits and its epilogue turns each accumulator tile
into ``dZ = g/T · (onehot − softmax)`` (bf16; the logits themselves are never written), then ``dH = dZ·W`` and
``dW += dZᵀ·H`` run on the tcgen05 GEMM with the operands read as stored and fp32 accumulation of ``dW`` in the epilogue.
Reference (CPU + oracle): chunked fp32 ``x[target]/T − logsumexp(x/T)``, as the reference framework does in
``unirl/models/qwen3/ar.py:74-99`` with ``torch.utils.checkpoint``.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from unirl_b200.ops._ext import count_launch, ext, require_ext, use_native

_BWD_CHUNK = int(os.environ.get("UNIRL_B200_LOGPROB_BWD_CHUNK", "8192"))


def linear_logprob_reference(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                             chunk: int = 2048) -> torch.Tensor:
    outs = []
    for s in range(0, hidden.shape[0], chunk):
        z = (hidden[s : s + chunk].float() @ weight.float().t()) / temperature
        outs.append(z.gather(-1, targets[s : s + chunk].long().unsqueeze(-1)).squeeze(-1) - torch.logsumexp(z, -1))
    return torch.cat(outs) if outs else hidden.new_zeros(0, dtype=torch.float32)


class _LinearLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, temperature):
        C = require_ext()
        hidden = hidden.contiguous()
        tgt = targets.to(torch.int32).contiguous()
        logp, lse = C.linear_logprob_fwd(hidden, weight, tgt, float(temperature))
        count_launch(2)
        ctx.save_for_backward(hidden, weight, tgt, lse)
        ctx.temperature = float(temperature)
        # set by the sharded trainer on its parameters: returns the fp32 gradient-accumulator view of this weight
        # (not for a weight that also receives gradient from another use, e.g. tied input embeddings: `_wgrad_shared`)
        fuse = os.environ.get("UNIRL_B200_WGRAD_FUSION", "1") != "0" and not getattr(weight, "_wgrad_shared", False)
        ctx.accum = getattr(weight, "_wgrad_accum", None) if fuse else None
        ctx.param = weight if ctx.accum is not None else None
        return logp

    @staticmethod
    def backward(ctx, g):
        C = require_ext()
        hidden, weight, tgt, lse = ctx.saved_tensors
        g = g.float().contiguous()
        d_hidden = torch.empty_like(hidden)
        # dW accumulates in fp32 INSIDE the GEMM (C = C + dZᵀ·H with fp32 output): chunk after chunk, and -- when the trainer
        # exposes its accumulator -- straight into that buffer, so no [V, H] gradient is converted, added or copied afterwards.
        fused_into_trainer = ctx.needs_input_grad[1] and ctx.accum is not None
        d_weight = None
        if ctx.needs_input_grad[1]:
            d_weight = ctx.accum() if fused_into_trainer else torch.zeros_like(weight, dtype=torch.float32)
        native = (os.environ.get("UNIRL_B200_GEMM_BWD", "native") == "native" and hasattr(C, "linear_dlogits") and weight.shape[0] % 8 == 0
                  and weight.is_contiguous())
        for s in range(0, hidden.shape[0], _BWD_CHUNK):
            e = min(s + _BWD_CHUNK, hidden.shape[0])
            h = hidden[s:e]
            if native:
                z = C.linear_dlogits(h, weight, tgt[s:e], lse[s:e], g[s:e], ctx.temperature, 0)  # dZ from the recompute GEMM's epilogue
                C.gemm_bf16(z, weight, False, True, d_hidden[s:e], False)  # dH = dZ·W
                if d_weight is not None:
                    C.gemm_bf16(z, h, True, True, d_weight, True)  # dW += dZᵀ·H
                count_launch(3)
                continue
            z = h @ weight.t()  # bf16 scratch [chunk, V]
            C.logprob_dlogits_inplace(z, tgt[s:e], lse[s:e], g[s:e], ctx.temperature)
            count_launch()
            torch.matmul(z, weight, out=d_hidden[s:e])
            if d_weight is not None:
                torch.addmm(d_weight, z.t(), h, out_dtype=torch.float32, out=d_weight)
        if fused_into_trainer:
            ctx.param._wgrad_fused = True
            return d_hidden, torch.empty(weight.shape, dtype=weight.dtype, device=weight.device), None, None
        return d_hidden, (d_weight.to(weight.dtype) if d_weight is not None else None), None, None


def linear_logprob(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    """fp32 ``[T]`` log-probs of ``targets`` under ``softmax(hidden·weightᵀ / temperature)``."""
    if use_native(hidden) and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and hidden.shape[1] % 8 == 0:
        return _LinearLogprob.apply(hidden, weight, targets, temperature)
    return _CheckpointedReference.apply(hidden, weight, targets, float(temperature))


class _CheckpointedReference(torch.autograd.Function):
    """CPU path: recompute each vocab projection chunk in backward instead of storing ``[T, V]``."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, temperature):
        ctx.save_for_backward(hidden, weight, targets)
        ctx.temperature = temperature
        with torch.no_grad():
            return linear_logprob_reference(hidden, weight, targets, temperature)

    @staticmethod
    def backward(ctx, g):
        hidden, weight, targets = ctx.saved_tensors
        t = ctx.temperature
        dh = torch.zeros_like(hidden, dtype=torch.float32)
        dw = torch.zeros_like(weight, dtype=torch.float32)
        wf = weight.float()
        for s in range(0, hidden.shape[0], 2048):
            h = hidden[s : s + 2048].float()
            p = torch.softmax((h @ wf.t()) / t, -1)
            dz = -p
            dz.scatter_add_(-1, targets[s : s + 2048].long().unsqueeze(-1), torch.ones_like(dz[:, :1]))
            dz *= (g[s : s + 2048].float() / t).unsqueeze(-1)
            dh[s : s + 2048] = dz @ wf
            dw += dz.t() @ h
        return dh.to(hidden.dtype), dw.to(weight.dtype), None, None


__all__ = ["linear_logprob", "linear_logprob_reference"]
