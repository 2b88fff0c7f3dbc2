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
from typing import Optional, Sequence, Tuple

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


# ------------------------------------------------------------------------------------------------ packed sequences (AR replay)
class PackedPlan:
    """Placement of a packed micro-batch of sequences (lengths ``lens``) on one context-parallel rank.

    Every sequence is cut into ``P`` chunks of ``n_i = ceil(L_i / P)`` tokens (the last chunks padded); rank ``r`` holds chunk ``r`` of
    every sequence, packed sequence after sequence, so all ranks hold ``Σ n_i`` tokens.  Keys and values are all-gathered (rank-major) and
    re-indexed per rank into, for every sequence, the chunks ``0 .. r`` in global order: exactly the prefix its queries may see, so the
    attention is a packed causal attention with ``n_i`` queries against ``(r + 1) · n_i`` keys, aligned at the end (the convention of the
    flash kernels).  Padding sits at the tail of a sequence, after every real token, and is never attended to by one.
    """

    def __init__(self, lens: Sequence[int], size: int, rank: int):
        self.lens, self.size, self.rank = [int(n) for n in lens], int(size), int(rank)
        self.chunk = [-(-n // self.size) for n in self.lens]
        self.local_tokens = sum(self.chunk)
        offs, idx, o = [], [], 0
        for n in self.chunk:
            offs.append(o)
            o += n
        self.offsets = offs
        for i, n in enumerate(self.chunk):
            for s in range(self.rank + 1):
                idx.append(torch.arange(n) + s * self.local_tokens + offs[i])
        self.kv_index = torch.cat(idx) if idx else torch.zeros(0, dtype=torch.long)
        self.cu_q = torch.tensor([0] + list(torch.tensor(self.chunk).cumsum(0).tolist()), dtype=torch.int32)
        self.cu_k = self.cu_q * (self.rank + 1)

    def local_slice(self, seq: torch.Tensor, i: int, pad: int = 0) -> torch.Tensor:
        """Chunk ``rank`` of sequence ``i`` (a 1-D tensor of its ``L_i`` tokens), padded to ``n_i``."""
        n = self.chunk[i]
        part = seq[self.rank * n : (self.rank + 1) * n]
        return part if part.numel() == n else torch.cat([part, part.new_full((n - part.numel(),), pad)])

    def local_positions(self) -> torch.Tensor:
        return torch.cat([torch.arange(n) + self.rank * n for n in self.chunk]) if self.chunk else torch.zeros(0, dtype=torch.long)

    def locate(self, i: int, pos: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """For global positions ``pos`` of sequence ``i``: which of them this rank holds (bool mask) and their rows in the local stream."""
        n = self.chunk[i]
        mine = (pos >= self.rank * n) & (pos < (self.rank + 1) * n)
        return mine, pos[mine] - self.rank * n + self.offsets[i]


class _SumOverRanks(torch.autograd.Function):
    """Sum of per-rank partial vectors (each rank filled its own entries of a zero vector); the gradient of the sum reaches every rank whole."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        y = x.contiguous().clone()
        comm.all_reduce(y)
        return y

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        return g, None


def packed_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, plan: PackedPlan, comm: Comm, scale: float) -> torch.Tensor:
    """Causal attention of this rank's packed query chunks ``q [T_loc, Hq, D]`` against the prefixes of their sequences, keys / values
    ``[T_loc, Hkv, D]`` gathered over the group (differentiable: their gradients are summed over the ranks that read them)."""
    idx = plan.kv_index.to(q.device)
    kk = _GatherSeqSum.apply(k.unsqueeze(0), comm)[0].index_select(0, idx)
    vv = _GatherSeqSum.apply(v.unsqueeze(0), comm)[0].index_select(0, idx)
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        try:
            from flash_attn import flash_attn_varlen_func  # q and k of different lengths per sequence: the library kernel (causal mask aligned at the end)

            cq, ck = plan.cu_q.to(q.device), plan.cu_k.to(q.device)
            return flash_attn_varlen_func(q.contiguous(), kk.contiguous(), vv.contiguous(), cq, ck, max(plan.chunk), max(plan.chunk) * (plan.rank + 1), softmax_scale=float(scale),
                                          causal=True)
        except ImportError:
            pass
    out = torch.empty_like(q)
    cq, ck = plan.cu_q.tolist(), plan.cu_k.tolist()
    for i, n in enumerate(plan.chunk):
        if not n:
            continue
        qi, ki, vi = q[cq[i] : cq[i + 1]], kk[ck[i] : ck[i + 1]], vv[ck[i] : ck[i + 1]]
        mask = torch.arange(ki.shape[0], device=q.device)[None, :] <= (torch.arange(n, device=q.device)[:, None] + plan.rank * n)
        out[cq[i] : cq[i + 1]] = _masked_attention(qi.unsqueeze(0), ki.unsqueeze(0), vi.unsqueeze(0), mask, scale)[0]
    return out


__all__ = ["ContextParallel", "PackedPlan", "packed_attention", "reference_attention"]
