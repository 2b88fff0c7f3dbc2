"""Thin communicator over ``torch.distributed`` groups, degenerate-safe for world size 1.

Every collective the Python layer issues goes through a :class:`Comm` so the same role code runs
(a) in one process without any process group, (b) on CPU ranks over gloo, (c) one process per
B200 over NCCL/NVLink.  Ranks are *group-local*; ``global_ranks`` maps them to pool worker ids.
"""

from __future__ import annotations

import datetime
import os
from typing import Any, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


def default_backend(device: torch.device) -> str:
    return "cpu:gloo,cuda:nccl" if torch.device(device).type == "cuda" else "gloo"


def init_global_group(rank: int, world_size: int, addr: str, port: int, device: torch.device, timeout_s: float = 600.0) -> None:
    """Bring up the pool-wide default process group (idempotent)."""
    if dist.is_initialized() or world_size <= 1:
        return
    if torch.device(device).type == "cuda":
        torch.cuda.set_device(device)
    dist.init_process_group(
        backend=default_backend(device),
        init_method=f"tcp://{addr}:{port}",
        rank=rank,
        world_size=world_size,
        timeout=datetime.timedelta(seconds=timeout_s),
    )


class Comm:
    """Collectives over one process group (``group=None`` + ``size==1`` ⇒ all no-ops)."""

    def __init__(self, group: Optional[Any], global_ranks: Sequence[int], my_global_rank: int):
        self.group = group
        self.global_ranks = list(global_ranks)
        self.size = len(self.global_ranks)
        self.rank = self.global_ranks.index(my_global_rank) if my_global_rank in self.global_ranks else -1

    @classmethod
    def solo(cls) -> "Comm":
        return cls(None, [0], 0)

    @classmethod
    def world(cls) -> "Comm":
        if not dist.is_initialized():
            return cls.solo()
        n = dist.get_world_size()
        return cls(dist.group.WORLD, list(range(n)), dist.get_rank())

    @property
    def active(self) -> bool:
        return self.size > 1

    def _g(self, local_rank: int) -> int:
        return self.global_ranks[local_rank]

    def barrier(self) -> None:
        if self.active:
            dist.barrier(group=self.group)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.active:
            dist.broadcast(t, src=self._g(src), group=self.group)
        return t

    def all_reduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if self.active:
            rop = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
            dist.all_reduce(t, op=rop, group=self.group)
        return t

    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        if not self.active:
            return [t]
        out = [torch.empty_like(t) for _ in range(self.size)]
        dist.all_gather(out, t.contiguous(), group=self.group)
        return out

    def all_gather_into(self, out: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        if not self.active:
            out.copy_(t.view_as(out))
        else:
            dist.all_gather_into_tensor(out, t.contiguous(), group=self.group)
        return out

    def reduce_scatter_into(self, out: torch.Tensor, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        if not self.active:
            out.copy_(t.view_as(out))
            return out
        if t.device.type == "cpu":  # gloo has no reduce_scatter: emulate with all_reduce + slice
            tmp = t.clone()
            dist.all_reduce(tmp, group=self.group)
            out.copy_(tmp.view(self.size, -1)[self.rank].view_as(out))
            if op == "avg":
                out.div_(self.size)
            return out
        rop = dist.ReduceOp.AVG if op == "avg" else dist.ReduceOp.SUM
        dist.reduce_scatter_tensor(out, t.contiguous(), op=rop, group=self.group)
        return out

    def all_to_all_single(self, out: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        if not self.active:
            out.copy_(t)
        elif t.device.type == "cpu":
            parts_in = list(t.chunk(self.size, 0))
            gathered = [self.all_gather(p) for p in parts_in]  # gathered[j][r] = rank r's chunk j
            out.copy_(torch.cat([gathered[self.rank][r] for r in range(self.size)], 0))
        else:
            dist.all_to_all_single(out, t.contiguous(), group=self.group)
        return out

    def all_gather_object(self, obj: Any) -> List[Any]:
        if not self.active:
            return [obj]
        out: List[Any] = [None] * self.size
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def broadcast_object(self, obj: Any, src: int = 0) -> Any:
        if not self.active:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self._g(src), group=self.group)
        return box[0]

    def split(self, groups: Sequence[Sequence[int]]) -> "Comm":
        """Sub-communicator containing this rank; ``groups`` partition the members by GROUP-LOCAL rank.

        Only the members of a sub-group take part in creating it (local synchronisation), so
        different sub-groups can be built concurrently.
        """
        mine = next((list(g) for g in groups if self.rank in g), None)
        if mine is None:
            raise ValueError(f"rank {self.rank} is in none of the sub-groups {groups}")
        globals_ = [self.global_ranks[r] for r in mine]
        if len(mine) == 1 or not self.active:
            return Comm(None, globals_, self.global_ranks[self.rank])
        g = dist.new_group(ranks=globals_, use_local_synchronization=True)
        return Comm(g, globals_, self.global_ranks[self.rank])

    # p2p takes GLOBAL worker ids (the transport plans hops between arbitrary pool workers)
    def send(self, t: torch.Tensor, dst_global: int) -> None:
        dist.send(t.contiguous(), dst=dst_global, group=self.group)

    def recv(self, t: torch.Tensor, src_global: int) -> None:
        dist.recv(t, src=src_global, group=self.group)


class MailboxComm:
    """p2p for several inline workers living in ONE process: a shared dict instead of a wire."""

    _boxes: Dict[tuple, List[torch.Tensor]] = {}

    def __init__(self, my_global_rank: int):
        self.me = my_global_rank

    def send(self, t: torch.Tensor, dst_global: int) -> None:
        MailboxComm._boxes.setdefault((self.me, dst_global), []).append(t)

    def recv(self, t: torch.Tensor, src_global: int) -> None:
        t.copy_(MailboxComm._boxes[(src_global, self.me)].pop(0))


__all__ = ["Comm", "MailboxComm", "init_global_group", "default_backend"]
