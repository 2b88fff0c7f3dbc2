"""Expert parallelism for mixture-of-experts feed-forward layers.

Every rank of the expert group owns ``E / P`` of a layer's routed experts.  Dispatch and combine use the two collectives
that are exact and bandwidth-cheap on an NVSwitch node:

* dispatch — **all-gather** of the tokens (and of their routing decisions, recomputed locally from the gathered tokens since
  the router is replicated): every rank sees every token and runs ITS experts on the tokens routed to them;
* combine — **reduce-scatter (sum)** of the per-rank partial outputs: each rank ends with the combined outputs of its own
  tokens.

Backward mirrors it (all-gather ↔ reduce-scatter).  Expert parameters are *not* replicated: the sharded trainer keeps them
in groups of their own that skip the data-parallel reduction; their gradient already sums over every rank's tokens and is
scaled by ``1 / P`` to match the rank-averaged objective.

Parity: the ``ep`` field of ``RankInfo`` / ``TrainTopology`` (``unirl/distributed/group/remote.py:21-39``,
``unirl/train/backend/base.py:38-91``) and the expert-parallel degree the reference passes to its external engines
(``unirl/rollout/engine/vllm_omni/stage_configs/hunyuan_image3_t2i_rl.yaml:46,92-98``).
"""

from __future__ import annotations

from typing import Any, List

import torch

from unirl_b200.distributed.group.comm import Comm


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm, ctx.n = comm, x.shape[0]
        out = x.new_empty(comm.size * x.shape[0], *x.shape[1:])
        comm.all_gather_into(out, x.contiguous())
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        out = g.new_empty(ctx.n, *g.shape[1:])
        ctx.comm.reduce_scatter_into(out, g.contiguous(), op="sum")
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Comm) -> torch.Tensor:
        ctx.comm = comm
        out = x.new_empty(x.shape[0] // comm.size, *x.shape[1:])
        comm.reduce_scatter_into(out, x.contiguous(), op="sum")
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        out = g.new_empty(ctx.comm.size * g.shape[0], *g.shape[1:])
        ctx.comm.all_gather_into(out, g.contiguous())
        return out, None


class ExpertParallelContext:
    def __init__(self, comm: Comm):
        self.comm = comm
        self.size, self.rank = comm.size, max(comm.rank, 0)

    def local_experts(self, num_experts: int) -> List[int]:
        if num_experts % self.size:
            raise ValueError(f"{num_experts} experts do not split over {self.size} expert-parallel ranks")
        per = num_experts // self.size
        return list(range(self.rank * per, (self.rank + 1) * per))

    def gather_tokens(self, x: torch.Tensor) -> torch.Tensor:
        return _AllGatherRows.apply(x, self.comm)

    def combine(self, partial: torch.Tensor) -> torch.Tensor:
        return _ReduceScatterRows.apply(partial, self.comm)


def mark_expert_local(module: torch.nn.Module) -> None:
    """Tag the parameters of ``module`` as owned by this expert-parallel rank (not replicated across the expert group)."""
    for p in module.parameters():
        p._ep_local = True  # type: ignore[attr-defined]


__all__ = ["ExpertParallelContext", "mark_expert_local"]
