"""How a controller-side call is split over workers and how the results are merged.

``Dispatch`` decides the per-worker payload, ``Execute`` which workers run.  Role methods opt in
with ``@distributed``.  Unlike the reference — where ``dp_size`` always equals the world size —
handles here carry real ``tp``/``sp`` degrees (the native rollout engine is tensor-parallel and
the video DiT is sequence-parallel), so DP peers genuinely exist and receive identical shards.

Parity: ``unirl/distributed/group/dispatch.py:61-74`` (enums), ``:80-178`` (dispatch fns),
``:188-212`` (collect), ``:228-263`` (backward mode), ``:271-311`` (decorator).
"""

from __future__ import annotations

import functools
from enum import Enum, auto
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

from unirl_b200.distributed.tensor.pytree import pytree_cat, pytree_chunk
from unirl_b200.distributed.utils import Broadcast

Shard = Tuple[tuple, dict]
DISTRIBUTED_CONFIG_ATTR = "_distributed_config"


class Dispatch(Enum):
    BROADCAST = auto()  # identical payload everywhere
    SCATTER = auto()  # one shard per worker
    DP_SCATTER = auto()  # one shard per dp rank; tp/sp/pp peers share it
    DP_SCATTER_HEAD = auto()  # as DP_SCATTER but only the dp head gets data


class Execute(Enum):
    ALL = auto()
    RANK_ZERO = auto()


def _strip(args: tuple, kwargs: dict) -> Shard:
    un = lambda v: v.value if isinstance(v, Broadcast) else v  # noqa: E731
    return tuple(un(a) for a in args), {k: un(v) for k, v in kwargs.items()}


def _split(args: tuple, kwargs: dict, parts: int, batch_size: int) -> List[Shard]:
    a_cols = [pytree_chunk(v, parts, batch_size) for v in args]
    k_cols = {k: pytree_chunk(v, parts, batch_size) for k, v in kwargs.items()}
    return [(tuple(c[i] for c in a_cols), {k: c[i] for k, c in k_cols.items()}) for i in range(parts)]


def is_dp_head(ri: Any) -> bool:
    return ri.tp_rank == 0 and ri.pp_rank == 0 and ri.sp_rank == 0


def plan_dispatch(mode: Dispatch, rank_infos: Sequence[Any], dp_size: int, args: tuple, kwargs: dict, batch_size: Optional[int]) -> List[Shard]:
    """Per-worker ``(args, kwargs)`` for one call."""
    world = len(rank_infos)
    if mode is Dispatch.BROADCAST or batch_size is None:
        whole = _strip(args, kwargs)
        if mode is Dispatch.DP_SCATTER_HEAD:
            return [whole if is_dp_head(ri) else ((), {}) for ri in rank_infos]
        return [whole] * world
    if mode is Dispatch.SCATTER:
        return _split(args, kwargs, world, batch_size)
    shards = _split(args, kwargs, dp_size, batch_size)
    if mode is Dispatch.DP_SCATTER:
        return [shards[ri.dp_rank] for ri in rank_infos]
    if mode is Dispatch.DP_SCATTER_HEAD:
        return [shards[ri.dp_rank] if is_dp_head(ri) else ((), {}) for ri in rank_infos]
    raise ValueError(mode)


def collect(mode: Dispatch, rank_infos: Sequence[Any], results: List[Any]) -> Any:
    """Merge per-worker results: raw list for BROADCAST/SCATTER, dp-head concat otherwise."""
    if mode in (Dispatch.BROADCAST, Dispatch.SCATTER):
        return results
    heads = [r for r, ri in zip(results, rank_infos) if ri.tp_rank == 0 and ri.is_pipeline_last_stage and ri.sp_rank == 0]
    if not heads:
        return None
    return heads[0] if len(heads) == 1 else pytree_cat(heads)


def resolve_backward_dispatch_mode(method_name: str, fwd: Dispatch, rank_infos: Sequence[Any]) -> Dispatch:
    """Backward RPCs always run DP_SCATTER on every rank; modes without a sample axis are rejected."""
    if fwd in (Dispatch.BROADCAST, Dispatch.SCATTER):
        raise ValueError(f"'{method_name}' is dispatched {fwd.name}: no shared sample axis, auto-backward unsupported")
    if any(ri.pp_size > 1 for ri in rank_infos):
        raise ValueError(f"'{method_name}' spans pp_size>1: auto-backward cannot cross pipeline stages")
    return Dispatch.DP_SCATTER


def distributed(_fn: Optional[Callable] = None, *, dispatch_mode: Dispatch = Dispatch.DP_SCATTER, execute_mode: Execute = Execute.ALL) -> Callable:
    """Mark a role method as callable through a :class:`Handle` (default ``DP_SCATTER`` / ``ALL``)."""

    def deco(fn: Callable) -> Callable:
        @functools.wraps(fn)
        def wrapper(*a: Any, **k: Any) -> Any:
            return fn(*a, **k)

        setattr(wrapper, DISTRIBUTED_CONFIG_ATTR, {"dispatch_mode": dispatch_mode, "execute_mode": execute_mode})
        return wrapper

    return deco(_fn) if _fn is not None else deco


def distributed_methods(cls: type) -> Dict[str, Dict[str, Any]]:
    out: Dict[str, Dict[str, Any]] = {}
    for name in dir(cls):
        cfg = getattr(getattr(cls, name, None), DISTRIBUTED_CONFIG_ATTR, None)
        if cfg is not None:
            out[name] = cfg
    return out


__all__ = [
    "Dispatch",
    "Execute",
    "distributed",
    "distributed_methods",
    "plan_dispatch",
    "collect",
    "is_dp_head",
    "resolve_backward_dispatch_mode",
    "DISTRIBUTED_CONFIG_ATTR",
]
