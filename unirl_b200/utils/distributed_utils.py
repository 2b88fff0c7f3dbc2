"""Extra process groups beside the default one, and a distributed masked whitening helper.

``init_process_group`` builds an additional *main* group from its own rendezvous (used by transports
that must not disturb the default group); ``distributed_masked_whiten`` normalises values with
statistics all-reduced as three floats.  Parity: ``unirl/utils/distributed_utils.py:39-117``, ``:120-154``.
"""

from __future__ import annotations

import datetime
from typing import Any, Optional

import torch
import torch.distributed as dist


def init_process_group(backend: str, init_method: str, world_size: int, rank: int, group_name: str = "extra", timeout_s: float = 600.0) -> Any:
    """A process group that is NOT the default one (own store, own ranks)."""
    from torch.distributed.distributed_c10d import _new_process_group_helper, rendezvous

    timeout = datetime.timedelta(seconds=timeout_s)
    store, rank, world_size = next(rendezvous(init_method, rank, world_size, timeout=timeout))
    store.set_timeout(timeout)
    store = dist.PrefixStore(group_name, store)
    pg, _ = _new_process_group_helper(world_size, rank, [], backend, store, group_name=group_name, timeout=timeout)
    return pg


def gloo_group(ranks: Optional[list] = None) -> Any:
    return dist.new_group(ranks=ranks, backend="gloo")


def distributed_masked_whiten(values: torch.Tensor, mask: torch.Tensor, group: Any = None, eps: float = 1e-8, shift_mean: bool = True) -> torch.Tensor:
    m = mask.to(values.dtype)
    stats = torch.stack([(values * m).sum(), (values.pow(2) * m).sum(), m.sum()]).float()
    if dist.is_initialized():
        dist.all_reduce(stats, group=group)
    mean = stats[0] / stats[2].clamp(min=1)
    var = (stats[1] / stats[2].clamp(min=1) - mean.pow(2)).clamp(min=0)
    out = (values - mean) * torch.rsqrt(var + eps)
    return out if shift_mean else out + mean


__all__ = ["init_process_group", "gloo_group", "distributed_masked_whiten"]
