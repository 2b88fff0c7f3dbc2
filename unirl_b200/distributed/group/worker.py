"""``Worker`` — one per device; hosts named roles, owns the tensor store, executes calls.

A worker is a plain object.  Three pool backends drive it: *inline* (same process), *mp* (one
spawned process per device, pipe RPC) and *spmd* (each ``torchrun`` rank owns one worker and
also runs the controller).  Parity: ``unirl/distributed/group/worker.py:37-88`` (construction),
``:189-267`` (``add_remote`` + nested ``_target_`` resolution), ``:275-331`` (``call``).
"""

from __future__ import annotations

import os
import threading
import time
import traceback
import uuid
from typing import Any, Dict, List, Optional, Sequence

import torch

from unirl_b200.config.instantiate import RESERVED, call_target, get_method
from unirl_b200.distributed.group.comm import Comm, MailboxComm, init_global_group
from unirl_b200.distributed.group.remote import RankInfo, Remote
from unirl_b200.distributed.tensor.transport import TensorMeta, TensorTransportRuntime, WorkerLocalTransport
from unirl_b200.distributed.utils import iter_leaves


class HandleRef:
    """Placeholder for "the co-located role named ``role_name``" inside init kwargs."""

    __slots__ = ("role_name",)

    def __init__(self, role_name: str):
        self.role_name = role_name

    def __repr__(self) -> str:
        return f"HandleRef({self.role_name!r})"

    def __reduce__(self):
        return (HandleRef, (self.role_name,))


def pick_device(worker_id: int, gpus_per_node: int = 8) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", worker_id % max(1, min(gpus_per_node, torch.cuda.device_count())))
    return torch.device("cpu")


class Worker:
    def __init__(self, worker_id: int, world_size: int, device: Optional[torch.device] = None, inline: bool = False):
        self.worker_id = worker_id
        self.world_size = world_size
        self.device = torch.device(device) if device is not None else pick_device(worker_id)
        if self.device.type == "cuda":
            if self.device.index is None:  # a bare "cuda" means the process's current device
                self.device = torch.device("cuda", torch.cuda.current_device())
            torch.cuda.set_device(self.device)
        self.inline = inline
        self._roles: Dict[str, Remote] = {}
        self._groups: Dict[str, Comm] = {}
        p2p = MailboxComm(worker_id) if inline else None
        self.transport = WorkerLocalTransport(worker_id, self.device, p2p)
        if not inline:
            TensorTransportRuntime.install(self.transport)
        self.heartbeat = time.time()

    # ---- process groups ------------------------------------------------------------------------
    def setup_global_pg(self, addr: str, port: int, timeout_s: float = 600.0) -> None:
        init_global_group(self.worker_id, self.world_size, addr, port, self.device, timeout_s)
        if self.world_size > 1:
            self.transport.comm = Comm.world()

    def new_group(self, tag: str, ranks: Sequence[int]) -> None:
        """Collective over ALL pool workers (``torch.distributed.new_group`` contract)."""
        import torch.distributed as dist

        ranks = list(ranks)
        if len(ranks) <= 1 or not dist.is_initialized():
            self._groups[tag] = Comm(None, ranks, self.worker_id) if self.worker_id in ranks else Comm.solo()
            return
        g = dist.new_group(ranks=ranks)
        if self.worker_id in ranks:
            self._groups[tag] = Comm(g, ranks, self.worker_id)

    # ---- roles ----------------------------------------------------------------------------------
    def _materialize(self, value: Any) -> Any:
        """Depth-first: ``HandleRef`` → sibling role; ``{_target_: …}`` → constructed object."""
        if isinstance(value, HandleRef):
            return self._roles[value.role_name]
        if isinstance(value, dict):
            built = {k: self._materialize(v) for k, v in value.items() if k not in RESERVED}
            if "_target_" in value:
                return call_target(get_method(value["_target_"]), **built)
            return built
        if isinstance(value, list):
            return [self._materialize(v) for v in value]
        return value

    def add_remote(self, role_name: str, target: Any, init_kwargs: Dict[str, Any], rank_info: RankInfo,
                   dist_env: Dict[str, str], group_tag: Optional[str] = None) -> None:
        factory = get_method(target) if isinstance(target, str) else target
        role = factory(**{k: self._materialize(v) for k, v in init_kwargs.items()})
        if not isinstance(role, Remote):
            raise TypeError(f"role '{role_name}': {target} did not produce a Remote (got {type(role).__name__})")
        comm = self._groups.get(group_tag) if group_tag else None
        role.setup(self.transport, str(self.device), rank_info, dist_env, self._roles.__getitem__, comm)
        self._roles[role_name] = role

    def remove_remote(self, role_name: str) -> None:
        self._roles.pop(role_name, None)

    def has_role(self, role_name: str) -> bool:
        return role_name in self._roles

    def get_role(self, role_name: str) -> Remote:
        return self._roles[role_name]

    def rank_info(self, role_name: str) -> RankInfo:
        return self._roles[role_name].rank_info

    # ---- calls ----------------------------------------------------------------------------------
    def call(self, role_name: str, method: str, args: tuple, kwargs: dict, grad_mode: bool = False,
             call_id: Optional[str] = None) -> Any:
        role = self._roles[role_name]
        prev = TensorTransportRuntime.current()
        TensorTransportRuntime.install(self.transport)
        try:
            args, kwargs = self.transport.hydrate((tuple(args), dict(kwargs)))
            if grad_mode:
                ins = [t for _, t, _ in iter_leaves([list(args), kwargs], torch.Tensor) if t.is_floating_point()]
                for t in ins:
                    if t.is_leaf:
                        t.requires_grad_(True)
                role._grad_inputs[call_id] = ins
                with torch.enable_grad():
                    out = getattr(role, method)(*args, **kwargs)
                role._grad_outputs[call_id] = [t for _, t, _ in iter_leaves([out], torch.Tensor)]
            else:
                out = getattr(role, method)(*args, **kwargs)
            return self.transport.dehydrate(out)
        finally:
            self.transport.end_call()
            self.heartbeat = time.time()
            TensorTransportRuntime.install(prev)

    def transport_op(self, op: str, *args: Any) -> Any:
        return self.transport.remote_op(op, *args)

    def ping(self) -> float:
        self.heartbeat = time.time()
        return self.heartbeat

    def shutdown(self) -> None:
        self._roles.clear()
        self.transport.clear()


def worker_main(conn: Any, worker_id: int, world_size: int, device_str: Optional[str], env: Dict[str, str]) -> None:
    """Entry point of an *mp* backend worker process: serve ``(req_id, op, args)`` requests until ``shutdown``."""
    os.environ.update(env)
    try:
        torch.set_num_threads(max(1, int(env.get("UNIRL_WORKER_THREADS", "2"))))
        device = torch.device(device_str) if device_str else pick_device(worker_id)
        w = Worker(worker_id, world_size, device)
    except BaseException:  # noqa: BLE001
        conn.send((0, False, traceback.format_exc()))
        return
    conn.send((0, True, str(w.device)))
    while True:
        try:
            req_id, op, args = conn.recv()
        except (EOFError, OSError):
            break
        try:
            if op == "shutdown":
                w.shutdown()
                conn.send((req_id, True, None))
                break
            res = getattr(w, op)(*args)
            conn.send((req_id, True, res))
        except BaseException:  # noqa: BLE001 - every failure must reach the controller
            conn.send((req_id, False, traceback.format_exc()))
    try:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        pass


__all__ = ["Worker", "HandleRef", "worker_main", "pick_device"]
