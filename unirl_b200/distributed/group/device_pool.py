"""``DevicePool`` — the set of workers (one per device) a job runs on, behind three backends.

* ``inline`` – workers are objects in the controller process (tests, single GPU).
* ``mp``     – the controller spawns one process per device and talks over pipes; workers form a
               ``torch.distributed`` world (gloo on CPU, NCCL on B200s).  This replaces the
               reference's Ray actors + placement groups (``device_pool.py:32-257``) on one box.
* ``spmd``   – launched by ``torchrun``: each rank hosts worker ``RANK`` *and* runs the same
               controller program; calls execute on the local shard and metadata is
               all-gathered, so there is no RPC hop at all (one process per GPU end to end).

Failure detection (host only): every controller→worker request carries a deadline; a dead or
silent worker raises :class:`WorkerTimeout` / :class:`WorkerDied` naming worker and operation.
"""

from __future__ import annotations

import itertools
import multiprocessing as mp
import os
import time
import weakref
from typing import Any, Callable, Dict, List, Optional, Sequence, Set, Tuple

import torch

from unirl_b200.distributed.group.comm import Comm, init_global_group
from unirl_b200.distributed.group.worker import Worker, pick_device, worker_main
from unirl_b200.distributed.tensor.transport import TensorMeta, TensorRef, TensorTransport, TensorTransportRuntime
from unirl_b200.distributed.utils import free_port, iter_leaves


class WorkerError(RuntimeError):
    """A role method raised on a worker; the message carries the remote traceback."""


class WorkerTimeout(TimeoutError):
    pass


class WorkerDied(RuntimeError):
    pass


class _Done:
    def __init__(self, value: Any = None, error: Optional[str] = None):
        self.value, self.error = value, error

    def result(self, timeout: Optional[float] = None) -> Any:
        if self.error is not None:
            raise WorkerError(self.error)
        return self.value


class _InlineProxy:
    def __init__(self, worker: Worker):
        self.worker = worker

    def submit(self, op: str, *args: Any) -> _Done:
        import traceback

        try:
            return _Done(getattr(self.worker, op)(*args))
        except Exception:  # noqa: BLE001
            return _Done(error=traceback.format_exc())

    def close(self) -> None:
        self.worker.shutdown()


class _PipeFuture:
    def __init__(self, proxy: "_PipeProxy", req_id: int, what: str):
        self.proxy, self.req_id, self.what = proxy, req_id, what

    def result(self, timeout: Optional[float] = None) -> Any:
        return self.proxy.wait(self.req_id, self.what, timeout)


class _PipeProxy:
    def __init__(self, worker_id: int, conn: Any, proc: Any, default_timeout: float):
        self.worker_id, self.conn, self.proc = worker_id, conn, proc
        self.default_timeout = default_timeout
        self._ids = itertools.count(1)
        self._ready: Dict[int, Any] = {}

    def submit(self, op: str, *args: Any) -> _PipeFuture:
        rid = next(self._ids)
        try:
            self.conn.send((rid, op, args))
        except (BrokenPipeError, OSError) as e:
            raise WorkerDied(f"worker {self.worker_id} is gone (sending '{op}'): {e}") from None
        what = f"{op}:{args[0]}.{args[1]}" if op == "call" else op
        return _PipeFuture(self, rid, what)

    def wait(self, rid: int, what: str, timeout: Optional[float]) -> Any:
        deadline = time.time() + (self.default_timeout if timeout is None else timeout)
        while rid not in self._ready:
            left = deadline - time.time()
            if left <= 0:
                raise WorkerTimeout(f"worker {self.worker_id} did not answer '{what}' within its deadline")
            if self.conn.poll(min(left, 0.5)):
                try:
                    got_id, ok, payload = self.conn.recv()
                except (EOFError, OSError):
                    raise WorkerDied(f"worker {self.worker_id} closed its pipe during '{what}'") from None
                self._ready[got_id] = (ok, payload)
            elif not self.proc.is_alive():
                raise WorkerDied(f"worker {self.worker_id} exited (code {self.proc.exitcode}) during '{what}'")
        ok, payload = self._ready.pop(rid)
        if not ok:
            raise WorkerError(f"worker {self.worker_id} failed in '{what}':\n{payload}")
        return payload

    def close(self) -> None:
        try:
            if self.proc.is_alive():
                self.submit("shutdown").result(10.0)
        except Exception:  # noqa: BLE001
            pass
        self.proc.join(5.0)
        if self.proc.is_alive():
            self.proc.kill()


class _ControllerTransport(TensorTransport):
    """Transport view for code running on the controller: fetches rows from the owning workers."""

    def __init__(self, pool: "DevicePool"):
        self.pool = pool

    def put(self, tensor: torch.Tensor) -> TensorRef:
        raise RuntimeError("the controller does not store tensors; return them from a role method instead")

    def get(self, refs: Sequence[TensorRef]) -> torch.Tensor:
        return self.pool.fetch(refs)

    def free(self, ref: TensorRef) -> None:
        self.pool.release(ref)

    def dehydrate(self, tree: Any) -> Any:
        return tree


class _SpmdTransport(TensorTransport):
    """Transport of a process that is both controller and worker (one per GPU under ``torchrun``).

    Inside a role method it is the worker's own store.  In controller code (which every rank runs identically) a
    handle owned by another rank is fetched collectively, exactly like the dedicated controller would.
    """

    def __init__(self, pool: "DevicePool", inner: TensorTransport):
        self.pool, self.inner = pool, inner

    def __getattr__(self, name: str) -> Any:
        return getattr(self.inner, name)

    def put(self, tensor: torch.Tensor) -> TensorRef:
        return self.inner.put(tensor)

    def get(self, refs: Sequence[TensorRef]) -> torch.Tensor:
        if self.pool._worker_depth == 0 and any(r.owner != self.inner.worker_id for r in refs):
            return self.pool.fetch(refs)
        return self.inner.get(refs)

    def free(self, ref: TensorRef) -> None:
        self.inner.free(ref)

    def end_call(self) -> None:
        self.inner.end_call()


class DevicePool:
    def __init__(self, num_nodes: int = 1, gpus_per_node: Optional[int] = None, backend: Optional[str] = None,
                 tensor_transport: str = "colocate_store", call_timeout_s: float = 3600.0, device: Optional[str] = None,
                 workers_per_device: int = 1, **_unused: Any):
        if num_nodes != 1:
            raise NotImplementedError("one NVSwitch domain (a single 8xB200 node) is the supported topology")
        spmd_env = "RANK" in os.environ and "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1
        self.backend = backend or ("spmd" if spmd_env else "inline")
        if gpus_per_node is None:
            gpus_per_node = int(os.environ.get("WORLD_SIZE", 0)) if self.backend == "spmd" else 0
            gpus_per_node = gpus_per_node or max(1, torch.cuda.device_count())
        self.num_devices = int(gpus_per_node)
        self.tensor_transport = tensor_transport
        self.call_timeout_s = float(call_timeout_s)
        self._claimed: Set[int] = set()
        self._role_counter: Dict[str, int] = {}
        self._handles: List[Any] = []
        self._group_tags = itertools.count(1)
        self.my_rank = 0
        self.workers: List[Any] = []
        self.local_worker: Optional[Worker] = None
        self.world_comm = Comm.solo()
        self._force_device = device
        self._worker_depth = 0  # > 0 while this process executes a role method (spmd: controller and worker share the process)
        getattr(self, f"_start_{self.backend}")()
        TensorTransportRuntime.install(_ControllerTransport(self) if self.backend != "spmd" else _SpmdTransport(self, self.local_worker.transport))

    # ---- bring-up --------------------------------------------------------------------------------
    def _dev(self, i: int) -> torch.device:
        return torch.device(self._force_device) if self._force_device else pick_device(i, self.num_devices)

    def _start_inline(self) -> None:
        self.workers = [_InlineProxy(Worker(i, self.num_devices, self._dev(i), inline=True)) for i in range(self.num_devices)]

    def _start_mp(self) -> None:
        ctx = mp.get_context("spawn")
        env = {"MASTER_ADDR": "127.0.0.1", "UNIRL_WORKER_THREADS": os.environ.get("UNIRL_WORKER_THREADS", "2")}
        for i in range(self.num_devices):
            parent, child = ctx.Pipe()
            dev = self._force_device or (None if torch.cuda.is_available() else "cpu")
            p = ctx.Process(target=worker_main, args=(child, i, self.num_devices, dev, env), daemon=True)
            p.start()
            child.close()
            self.workers.append(_PipeProxy(i, parent, p, self.call_timeout_s))
        for w in self.workers:  # first message = construction verdict
            w._ready[0] = None
            deadline = time.time() + 300
            while not w.conn.poll(0.5):
                if not w.proc.is_alive() or time.time() > deadline:
                    raise WorkerDied(f"worker {w.worker_id} failed to start")
            _rid, ok, payload = w.conn.recv()
            w._ready.pop(0, None)
            if not ok:
                raise WorkerError(f"worker {w.worker_id} failed to start:\n{payload}")
        if self.num_devices > 1:
            port = free_port()
            futs = [w.submit("setup_global_pg", "127.0.0.1", port, self.call_timeout_s) for w in self.workers]
            for f in futs:
                f.result(300.0)

    def _start_spmd(self) -> None:
        self.my_rank = int(os.environ["RANK"])
        world = int(os.environ["WORLD_SIZE"])
        self.num_devices = world
        local = int(os.environ.get("LOCAL_RANK", self.my_rank))
        dev = torch.device(self._force_device) if self._force_device else (
            torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu"))
        init_global_group(self.my_rank, world, os.environ.get("MASTER_ADDR", "127.0.0.1"),
                          int(os.environ.get("MASTER_PORT", "29500")), dev, self.call_timeout_s)
        self.local_worker = Worker(self.my_rank, world, dev)
        self.world_comm = Comm.world()
        self.local_worker.transport.comm = self.world_comm
        self.workers = [None] * world

    # ---- placement bookkeeping ---------------------------------------------------------------------
    def allocate(self, n: int) -> List[int]:
        free = [i for i in range(self.num_devices) if i not in self._claimed]
        if len(free) < n:
            raise RuntimeError(f"pool exhausted: asked for {n} devices, {len(free)} unclaimed")
        got = free[:n]
        self._claimed.update(got)
        return got

    def unique_role_name(self, base: str) -> str:
        k = self._role_counter.get(base, 0)
        self._role_counter[base] = k + 1
        return base if k == 0 else f"{base}_{k}"

    def get_workers(self, devices: Optional[Sequence[int]] = None) -> List[Any]:
        return [self.workers[i] for i in (devices if devices is not None else range(self.num_devices))]

    # ---- fan-out primitives used by Handle ------------------------------------------------------------
    def run_on(self, devices: Sequence[int], op: str, per_worker_args: Sequence[tuple], timeout: Optional[float] = None) -> List[Any]:
        """Run ``Worker.<op>(*args_i)`` on ``devices[i]``; results in device order on every controller."""
        if self.backend == "spmd":
            mine, err = None, None
            if self.my_rank in devices:
                import traceback

                self._worker_depth += 1
                try:
                    mine = getattr(self.local_worker, op)(*per_worker_args[list(devices).index(self.my_rank)])
                except Exception:  # noqa: BLE001
                    err = traceback.format_exc()
                finally:
                    self._worker_depth -= 1
            gathered = self.world_comm.all_gather_object((mine, err))
            for r in devices:
                if gathered[r][1] is not None:
                    raise WorkerError(f"worker {r} failed in '{op}':\n{gathered[r][1]}")
            return [gathered[r][0] for r in devices]
        futs = [self.workers[d].submit(op, *a) for d, a in zip(devices, per_worker_args)]
        errors, out = [], []
        for f in futs:
            try:
                out.append(f.result(timeout))
            except (WorkerError, WorkerTimeout, WorkerDied) as e:
                errors.append(e)
                out.append(None)
        if errors:
            raise errors[0]
        return out

    def run_many(self, calls: Sequence[tuple], timeout: Optional[float] = None) -> List[List[Any]]:
        """Several fan-outs in flight at once: ``calls = [(devices, op, per_worker_args), …]``.

        Needed when roles on *different* workers must enter one collective together (trainer rank 0
        broadcasting weights while the engine ranks receive).  In spmd mode every rank runs the calls
        that target it, in order, and results are exchanged once at the end.
        """
        if self.backend == "spmd":
            import traceback

            mine: List[Any] = []
            err = None
            for devices, op, args in calls:
                res = None
                if self.my_rank in devices and err is None:
                    self._worker_depth += 1
                    try:
                        res = getattr(self.local_worker, op)(*args[list(devices).index(self.my_rank)])
                    except Exception:  # noqa: BLE001
                        err = traceback.format_exc()
                    finally:
                        self._worker_depth -= 1
                mine.append(res)
            gathered = self.world_comm.all_gather_object((mine, err))
            for r, (_m, e) in enumerate(gathered):
                if e is not None:
                    raise WorkerError(f"worker {r} failed in a concurrent call:\n{e}")
            return [[gathered[d][0][i] for d in devices] for i, (devices, _op, _a) in enumerate(calls)]
        if self.backend == "inline":
            return [self.run_on(devices, op, args, timeout) for devices, op, args in calls]
        futs = [[self.workers[d].submit(op, *a) for d, a in zip(devices, args)] for devices, op, args in calls]
        return [[f.result(timeout) for f in fl] for fl in futs]

    def run_everywhere(self, op: str, *args: Any) -> List[Any]:
        return self.run_on(list(range(self.num_devices)), op, [args] * self.num_devices)

    def new_group(self, ranks: Sequence[int]) -> str:
        tag = f"g{next(self._group_tags)}"
        self.run_everywhere("new_group", tag, list(ranks))
        return tag

    # ---- tensors -------------------------------------------------------------------------------------
    def move(self, hops: Sequence[tuple]) -> Dict[tuple, TensorRef]:
        """Execute ``(src, dst, ref)`` hops; returns ``{(*ref.ident, dst): new_ref}``."""
        mapping: Dict[tuple, TensorRef] = {}
        pairs: Dict[Tuple[int, int], List[TensorRef]] = {}
        for src, dst, ref in hops:  # everything between the same two workers travels together (one message per dtype)
            pairs.setdefault((src, dst), []).append(ref)
        for (src, dst), refs in pairs.items():
            if self.backend == "spmd":
                new = None
                if self.my_rank == src:
                    self.local_worker.transport.send_many(refs, dst)
                if self.my_rank == dst:
                    new = self.local_worker.transport.recv_many(refs, src)
                new = self.world_comm.broadcast_object(new, src=dst)
            elif self.backend == "inline":
                self.workers[src].submit("transport_op", "send_many", refs, dst).result()
                new = self.workers[dst].submit("transport_op", "recv_many", refs, src).result()
            else:
                fs = self.workers[src].submit("transport_op", "send_many", refs, dst)
                fr = self.workers[dst].submit("transport_op", "recv_many", refs, src)
                fs.result()
                new = fr.result()
            for ref, n in zip(refs, new):
                mapping[(*ref.ident, dst)] = self.adopt(n)
        return mapping

    def fetch(self, refs: Sequence[TensorRef]) -> torch.Tensor:
        """CPU copy of the rows behind ``refs`` on the controller (every controller in spmd mode)."""
        parts = []
        for r in refs:
            if self.backend == "spmd":
                t = self.local_worker.transport.get_cpu(r) if r.owner == self.my_rank else None
                parts.append(self.world_comm.broadcast_object(t, src=r.owner))
            else:
                parts.append(self.workers[r.owner].submit("transport_op", "get_cpu", r).result())
        if len(parts) == 1:
            return parts[0]
        return torch.stack(parts) if parts[0].dim() == 0 else torch.cat(parts, 0)

    def release(self, ref: TensorRef) -> None:
        try:
            if self.backend == "spmd":
                if ref.owner == self.my_rank:
                    self.local_worker.transport.decref(ref)
            elif self.workers and self.workers[ref.owner] is not None:
                self.workers[ref.owner].submit("transport_op", "decref", ref)
        except Exception:  # noqa: BLE001 - finalizers must never raise
            pass

    def adopt(self, ref: TensorRef) -> TensorRef:
        """Tie the stored tensor's lifetime to this controller-side ref object (windows ride on their parent)."""
        if ref.base is not None:
            return ref
        weakref.finalize(ref, DevicePool._release_static, weakref.ref(self), ref.owner, ref.key, ref.shape, ref.dtype, ref.device)
        return ref

    @staticmethod
    def _release_static(pool_ref: Any, owner: int, key: int, shape: tuple, dtype: Any, device: str) -> None:
        pool = pool_ref()
        if pool is not None and not pool._closed:
            pool.release(TensorRef(owner, key, shape, dtype, device))

    def adopt_tree(self, tree: Any) -> Any:
        for _p, meta, _s in iter_leaves(tree, TensorMeta):
            for r in meta.refs:
                if isinstance(r, TensorRef):
                    self.adopt(r)
        return tree

    def store_stats(self) -> List[Dict[str, int]]:
        return self.run_everywhere("transport_op", "stats")

    def reset_transfer_queue_buffers(self) -> None:
        """Per-rollout reclaim hook of the queue transport; the worker-local store frees by refcount."""

    def local_role(self, handle: Any) -> Any:
        """The role object behind ``handle`` when it lives in this process (inline and spmd pools), else ``None``.  For read-only
        inspection by the driver (metrics); calls still go through the handle."""
        lw = self.local_worker
        if lw is None and self.backend == "inline" and self.workers:
            lw = getattr(self.workers[0], "worker", None) or (self.workers[0] if hasattr(self.workers[0], "_roles") else None)
        return None if lw is None else getattr(lw, "_roles", {}).get(getattr(handle, "role_name", None))

    # ---- roles -----------------------------------------------------------------------------------------
    def create_remote(self, role_cls: Any, devices: Sequence[int], role_name: Optional[str] = None,
                      parallel: Optional[Dict[str, int]] = None, **init_kwargs: Any) -> Any:
        from unirl_b200.distributed.group.handle import Handle

        h = Handle(self, role_cls, list(devices), init_kwargs, role_name=role_name, parallel=parallel)
        self._handles.append(h)
        return h

    _closed = False

    def shutdown(self) -> None:
        if self._closed:
            return
        self._closed = True
        for w in self.workers:
            if w is not None:
                w.close()
        if self.backend == "spmd" and self.local_worker is not None:
            self.local_worker.shutdown()
        self.workers = []
        TensorTransportRuntime.install(None)

    def __enter__(self) -> "DevicePool":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.shutdown()


__all__ = ["DevicePool", "WorkerError", "WorkerTimeout", "WorkerDied"]
