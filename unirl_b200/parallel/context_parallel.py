"""Context parallelism for causal self-attention over long sequences: every rank holds a contiguous ``L / P`` slice of the
tokens; keys and values are all-gathered over the group (differentiably: the backward is a reduce-scatter of their gradients)
and each rank attends from ITS queries to the keys at or before them.

This is the all-gather variant (one collective per attention call, K / V of the whole sequence resident per layer), chosen
over a ring because one NVSwitch domain moves the gathered K / V of a 32 k-token sequence in tens of microseconds and the 180 GB
of HBM hold them easily; a ring only pays off across nodes.  Query shards late in the sequence see more keys than early
ones; :meth:`ContextParallel.shard_sequence` can deal the tokens in the zig-zag order (chunk ``r`` and chunk ``2P-1-r`` to rank
``r``) that evens the work out.

Parity: the reference only forwards ``ring_degree`` / ``cp_size`` knobs to its external engines
(``unirl/rollout/engine/vllm_omni/stage_configs/sd35_t2i_rl.yaml:47-49``, ``unirl/train/backend/base.py:54-56``).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from unirl_b200.distributed.group.comm import Comm


class _GatherSeqSum(torch.autograd.Function):
    """All-gather along the token axis; the gradient of every rank's slice is the SUM of what all ranks computed for it."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm, ctx.n = comm, x.shape[1]
        return torch.cat(comm.all_gather(x.contiguous()), 1)

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        g = g.contiguous().clone()
        ctx.comm.all_reduce(g)
        r = max(ctx.comm.rank, 0)
        return g[:, r * ctx.n : (r + 1) * ctx.n].contiguous(), None


class ContextParallel:
    def __init__(self, comm: Comm, zigzag: bool = False):
        self.comm = comm
        self.size, self.rank = comm.size, max(comm.rank, 0)
        self.zigzag = bool(zigzag) and self.size > 1

    # ---- token placement -------------------------------------------------------------------------------------------
    def token_index(self, length: int, rank: Optional[int] = None) -> torch.Tensor:
        """Global positions of the tokens rank ``rank`` holds (ascending)."""
        r = self.rank if rank is None else rank
        p = self.size
        if length % (2 * p if self.zigzag else p):
            raise ValueError(f"sequence of {length} tokens does not split over {p} context-parallel ranks")
        if not self.zigzag:
            n = length // p
            return torch.arange(r * n, (r + 1) * n)
        n = length // (2 * p)
        return torch.cat([torch.arange(r * n, (r + 1) * n), torch.arange((2 * p - 1 - r) * n, (2 * p - r) * n)])

    def shard_sequence(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        return x.index_select(dim, self.token_index(x.shape[dim]).to(x.device))

    def gather_sequence(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        """Inverse of :meth:`shard_sequence` (not differentiable; for outputs and tests)."""
        parts = self.comm.all_gather(x.contiguous())
        full = torch.cat(parts, dim)
        order = torch.cat([self.token_index(full.shape[dim], r) for r in range(self.size)])
        return full.index_select(dim, torch.argsort(order).to(x.device))

    # ---- attention -------------------------------------------------------------------------------------------------
    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
        """``q [B, l, Hq, D]``, ``k, v [B, l, Hkv, D]`` (this rank's tokens) → ``[B, l, Hq, D]``."""
        b, l, hq, d = q.shape
        scale = scale if scale is not None else 1.0 / math.sqrt(d)
        kk, vv = _GatherSeqSum.apply(k, self.comm), _GatherSeqSum.apply(v, self.comm)
        length = kk.shape[1]
        q_pos = self.token_index(length).to(q.device)
        k_pos = torch.cat([self.token_index(length, r) for r in range(self.size)]).to(q.device)  # order of the gathered keys
        mask = (k_pos[None, :] <= q_pos[:, None]) if causal else None
        return _masked_attention(q, kk, vv, mask, scale)


def _masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor], scale: float) -> torch.Tensor:
    import torch.nn.functional as F

    hq, hkv = q.shape[2], k.shape[2]
    qq, kk, vv = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if hq != hkv:
        kk, vv = kk.repeat_interleave(hq // hkv, 1), vv.repeat_interleave(hq // hkv, 1)
    o = F.scaled_dot_product_attention(qq, kk, vv, attn_mask=mask, scale=float(scale))
    return o.transpose(1, 2)


def reference_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Single-rank oracle on full sequences ``[B, L, H, D]``."""
    l = q.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    mask = torch.ones(l, l, dtype=torch.bool, device=q.device).tril() if causal else None
    return _masked_attention(q, k, v, mask, scale)


__all__ = ["ContextParallel", "reference_attention"]
