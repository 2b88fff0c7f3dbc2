"""``Handle`` — controller-side SPMD proxy for one role class on a list of devices.

For every ``@distributed`` method of the role class the handle exposes a same-named callable
that: validates the sample axis against ``dp_size``, plans per-worker payloads
(:func:`plan_dispatch`), moves foreign tensor rows to the consuming workers, fans the call out,
adopts returned handles (lifetime = controller references) and merges the results.

Parity: ``unirl/distributed/group/handle.py:94-107`` (``HandleRef``), ``:124-188`` (construction),
``:214-318`` (call path), ``:337-358`` (rebind).  Difference: ``parallel={"tp":…, "sp":…}`` gives
real tensor-/sequence-parallel rank layouts instead of hard-coding ``dp_size = world``.
"""

from __future__ import annotations

import uuid
from typing import Any, Dict, List, Optional, Sequence

from unirl_b200.distributed.group.dispatch import (
    Dispatch,
    Execute,
    collect,
    distributed_methods,
    plan_dispatch,
    resolve_backward_dispatch_mode,
)
from unirl_b200.distributed.group.remote import RankInfo, make_rank_infos
from unirl_b200.distributed.group.worker import HandleRef
from unirl_b200.distributed.tensor.pytree import infer_batch_size
from unirl_b200.distributed.tensor.transport import TensorMeta, plan_localize, rewrite_refs
from unirl_b200.distributed.utils import free_port, iter_leaves


def _owner_class(role_cls: Any) -> type:
    """The class whose ``@distributed`` methods define the proxy surface (factories are classmethods)."""
    if isinstance(role_cls, type):
        return role_cls
    owner = getattr(role_cls, "__self__", None)
    if isinstance(owner, type):
        return owner
    ret = getattr(role_cls, "__annotations__", {}).get("return")
    if isinstance(ret, type):
        return ret
    raise TypeError(f"cannot infer the role class behind {role_cls!r}; pass a class or a classmethod")


class Handle:
    def __init__(self, pool: Any, role_cls: Any, devices: List[int], init_kwargs: Dict[str, Any],
                 role_name: Optional[str] = None, parallel: Optional[Dict[str, int]] = None):
        self.pool = pool
        self.role_cls = role_cls
        self.cls = _owner_class(role_cls)
        self.devices = list(devices)
        self.world_size = len(self.devices)
        par = dict(parallel or {})
        self.rank_infos: List[RankInfo] = make_rank_infos(self.world_size, tp=par.get("tp", 1), sp=par.get("sp", 1),
                                                          pp=par.get("pp", 1), ep=par.get("ep", 1))
        self.dp_size = self.rank_infos[0].dp_size
        self.role_name = pool.unique_role_name(role_name or self.cls.__name__)
        self._grad_ctx = None
        port = free_port() if pool.my_rank == 0 else 0
        if pool.backend == "spmd":
            port = pool.world_comm.broadcast_object(port, 0)
        self.group_tag = pool.new_group(self.devices) if self.world_size > 1 else None
        kwargs = {k: (HandleRef(v.role_name) if isinstance(v, Handle) else v) for k, v in init_kwargs.items()}
        for k, v in init_kwargs.items():
            if isinstance(v, Handle) and not set(self.devices) <= set(v.devices):
                raise ValueError(f"role '{self.role_name}': sibling '{k}' ({v.role_name}) is not co-located on {self.devices}")
        per_worker = []
        for i, _d in enumerate(self.devices):
            env = {"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "WORLD_SIZE": str(self.world_size),
                   "RANK": str(i), "GROUP_NAME": self.role_name}
            per_worker.append((self.role_name, role_cls, kwargs, self.rank_infos[i], env, self.group_tag))
        pool.run_on(self.devices, "add_remote", per_worker)
        for name, cfg in distributed_methods(self.cls).items():
            setattr(self, name, self._bind(name, cfg["dispatch_mode"], cfg["execute_mode"]))

    # ------------------------------------------------------------------------------------------
    def _bind(self, method: str, mode: Dispatch, execute: Execute):
        def proxy(*args: Any, **kwargs: Any) -> Any:
            return self._invoke(method, mode, execute, args, kwargs)

        proxy.__name__ = method
        proxy.dispatch_mode, proxy.execute_mode = mode, execute
        return proxy

    def _invoke(self, method: str, mode: Dispatch, execute: Execute, args: tuple, kwargs: dict,
                timeout: Optional[float] = None) -> Any:
        bs = infer_batch_size(args, kwargs)
        if bs is not None and mode is not Dispatch.BROADCAST:
            parts = self.world_size if mode is Dispatch.SCATTER else self.dp_size
            if bs % parts:
                raise ValueError(f"{self.role_name}.{method}: batch of {bs} does not split over {parts} "
                                 f"{'workers' if mode is Dispatch.SCATTER else 'dp ranks'}")
        shards = plan_dispatch(mode, self.rank_infos, self.dp_size, args, kwargs, bs)
        devices, infos = self.devices, self.rank_infos
        if execute is Execute.RANK_ZERO:
            shards, devices, infos = shards[:1], devices[:1], infos[:1]
        hops = plan_localize(shards, devices)
        if hops:
            mapping = self.pool.move(hops)
            shards = [rewrite_refs(s, mapping, d) for s, d in zip(shards, devices)]
        ctx = self._grad_ctx
        call_id = uuid.uuid4().hex if ctx is not None else None
        if ctx is not None:
            resolve_backward_dispatch_mode(method, mode, self.rank_infos)
        payloads = [(self.role_name, method, a, k, ctx is not None, call_id) for a, k in shards]
        results = self.pool.run_on(devices, "call", payloads, timeout)
        self.pool.adopt_tree(results)
        out = collect(mode, infos, results)
        if ctx is not None:
            ctx.record(self, call_id, args, kwargs, out)
        return out

    def prepare(self, method: str, *args: Any, **kwargs: Any) -> tuple:
        """Plan a call without running it: returns ``(devices, "call", payloads)`` for ``pool.run_many``
        plus what :meth:`finish` needs.  No RPC autograd on this path."""
        cfg = getattr(getattr(self.cls, method), "_distributed_config", {"dispatch_mode": Dispatch.BROADCAST, "execute_mode": Execute.ALL})
        mode, execute = cfg["dispatch_mode"], cfg["execute_mode"]
        bs = infer_batch_size(args, kwargs)
        shards = plan_dispatch(mode, self.rank_infos, self.dp_size, args, kwargs, bs)
        devices, infos = self.devices, self.rank_infos
        if execute is Execute.RANK_ZERO:
            shards, devices, infos = shards[:1], devices[:1], infos[:1]
        hops = plan_localize(shards, devices)
        if hops:
            mapping = self.pool.move(hops)
            shards = [rewrite_refs(s, mapping, d) for s, d in zip(shards, devices)]
        payloads = [(self.role_name, method, a, k, False, None) for a, k in shards]
        return (devices, "call", payloads), (mode, infos)

    def finish(self, results: List[Any], ctx: tuple) -> Any:
        mode, infos = ctx
        self.pool.adopt_tree(results)
        return collect(mode, infos, results)

    def call(self, method: str, *args: Any, **kwargs: Any) -> Any:
        """Invoke a method that was not decorated (broadcast to all ranks, list of results)."""
        return self._invoke(method, Dispatch.BROADCAST, Execute.ALL, args, kwargs)

    def initialize(self, *args: Any, **kwargs: Any) -> "Handle":
        self._invoke("initialize", Dispatch.BROADCAST, Execute.ALL, args, kwargs)
        return self

    def remove(self) -> None:
        self.pool.run_on(self.devices, "remove_remote", [(self.role_name,)] * self.world_size)

    def __repr__(self) -> str:
        return f"Handle({self.role_name} on {self.devices}, dp={self.dp_size})"


def reset_role_name_counter(pool: Any) -> None:
    pool._role_counter.clear()


__all__ = ["Handle", "HandleRef", "reset_role_name_counter"]
