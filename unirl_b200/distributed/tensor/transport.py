"""Tensor transport: worker-resident tensor stores addressed by ``TensorMeta`` handles.

The controller never holds heavy tensors.  A role method's tensor outputs are *dehydrated* into
the executing worker's store and replaced by :class:`TensorMeta` handles; the next call that
receives such a handle *localizes* it (device-to-device hop when the owner differs) and
*hydrates* it back into a tensor on the consuming worker.

Classes
-------
``TensorRef``       one stored tensor: ``(owner worker, key, shape, dtype, device)``
``TensorMeta``      a ``Batch`` of refs along dim 0 (``sizes[i]`` rows per ref) with optional ``grad``
``TensorStore``     refcounted in-process dict (one per worker process)
``TensorTransport`` abstract contract (``put/get/put_batch/get_batch/dehydrate/hydrate/transform``)
``WorkerLocalTransport`` store-backed transport + peer send/recv and the ``localize`` planner

Parity: ``unirl/distributed/tensor/transport.py:40-163`` (TensorMeta), ``:285-441`` (ABC),
``:474-603`` (worker-local transport + localize).  One process per GPU means the CUDA-IPC store of
the reference (``backend/gpu_store``) collapses to pointer passing inside the worker process.
"""

from __future__ import annotations

import abc
import contextlib
import itertools
import threading
from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, shared_field
from unirl_b200.distributed.utils import map_leaves


@dataclass(frozen=True)
class TensorRef:
    """One stored tensor, or a window of ``shape[0]`` rows starting at row ``lo`` of it.

    A window keeps its parent ref object alive through ``base`` (the stored tensor's lifetime is tied to the
    parent object on the controller), so slicing a handle never copies and never frees early.
    """

    owner: int
    key: int
    shape: Tuple[int, ...]
    dtype: torch.dtype
    device: str
    lo: int = 0
    base: Optional["TensorRef"] = field(default=None, compare=False, repr=False)

    @property
    def rows(self) -> int:
        return int(self.shape[0]) if self.shape else 1

    def window(self, start: int, end: int) -> "TensorRef":
        if not self.shape:
            raise ValueError("a scalar ref has no rows to window")
        if not (0 <= start <= end <= self.rows):
            raise IndexError(f"window [{start}:{end}) outside {self.rows} rows")
        if start == 0 and end == self.rows:
            return self
        return TensorRef(self.owner, self.key, (end - start, *self.shape[1:]), self.dtype, self.device, self.lo + start, self.base or self)

    @property
    def ident(self) -> Tuple[int, int, int, int]:
        return (self.owner, self.key, self.lo, self.rows)


class TensorTransportRuntime:
    """Process-wide "current transport" slot (workers install theirs at start-up)."""

    _current: ClassVar[Optional["TensorTransport"]] = None

    @classmethod
    def install(cls, transport: Optional["TensorTransport"]) -> None:
        cls._current = transport

    @classmethod
    def current(cls) -> Optional["TensorTransport"]:
        return cls._current

    @classmethod
    def require(cls) -> "TensorTransport":
        if cls._current is None:
            raise RuntimeError("no TensorTransport installed in this process")
        return cls._current


@dataclass
class TensorMeta(Batch):
    """Handle to rows that live in worker stores.  ``batch_size == sum(sizes)``."""

    refs: List[Any] = concat_field(default_factory=list)
    sizes: List[int] = concat_field(default_factory=list)
    shape: Optional[Tuple[int, ...]] = shared_field(default=None)
    dtype: Optional[torch.dtype] = shared_field(default=None)
    device: Optional[str] = shared_field(default=None)
    grad: Optional["TensorMeta"] = shared_field(default=None)
    retain_grad_flag: bool = shared_field(default=False)

    @property
    def batch_size(self) -> int:
        return int(sum(self.sizes)) if self.sizes else 0

    def __len__(self) -> int:
        return self.batch_size

    def _with_refs(self, refs: List[Any], sizes: List[int]) -> "TensorMeta":
        total = int(sum(sizes))
        shape = (total, *self.shape[1:]) if self.shape else None
        return TensorMeta(refs=list(refs), sizes=[int(s) for s in sizes], shape=shape, dtype=self.dtype, device=self.device)

    @classmethod
    def concat(cls, items: Sequence["TensorMeta"]) -> "TensorMeta":
        items = list(items)
        refs = list(itertools.chain.from_iterable(m.refs for m in items))
        sizes = list(itertools.chain.from_iterable(m.sizes for m in items))
        return items[0]._with_refs(refs, sizes)

    @classmethod
    def from_refs(cls, refs: Sequence[TensorRef]) -> "TensorMeta":
        refs = list(refs)
        if not refs:
            return cls()
        sizes = [r.rows for r in refs]
        return cls(refs=refs, sizes=sizes, shape=(sum(sizes), *refs[0].shape[1:]), dtype=refs[0].dtype, device=refs[0].device)

    def select(self, indices):  # rows are remote: arbitrary gathers need the data
        raise NotImplementedError("TensorMeta.select: hydrate first")

    def slice(self, start: int, end: int) -> "TensorMeta":
        """Row range → the refs (whole, or windows of them) that cover it; no data moves."""
        start, end = max(0, int(start)), min(int(end), self.batch_size)
        refs, sizes, off = [], [], 0
        for r, n in zip(self.refs, self.sizes):
            a, b = max(start, off), min(end, off + int(n))
            if a < b:
                if a == off and b == off + int(n):
                    refs.append(r)
                elif isinstance(r, TensorRef):
                    refs.append(r.window(a - off, b - off))
                else:
                    raise NotImplementedError(f"TensorMeta rows [{start}:{end}) cut through a non-windowable ref {type(r).__name__}; hydrate first")
                sizes.append(b - a)
            off += int(n)
        return self._with_refs(refs, sizes)

    def __getitem__(self, key) -> "TensorMeta":
        if isinstance(key, slice) and key.step in (None, 1):
            return self.slice(key.start or 0, self.batch_size if key.stop is None else key.stop)
        raise NotImplementedError("TensorMeta supports contiguous slices only")

    def chunk_refs(self, n: int) -> List["TensorMeta"]:
        if len(self.refs) % n:
            raise ValueError(f"TensorMeta has {len(self.refs)} refs, not divisible by {n}")
        per = len(self.refs) // n
        return [self._with_refs(self.refs[i * per : (i + 1) * per], self.sizes[i * per : (i + 1) * per]) for i in range(n)]

    # ---- compute proxies ---------------------------------------------------------------------
    def transform(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "TensorMeta":
        return TensorTransportRuntime.require().transform(self, fn)

    def reshape(self, *shape: int) -> "TensorMeta":
        return self.transform(lambda t: t.reshape(*shape))

    def permute(self, *dims: int) -> "TensorMeta":
        return self.transform(lambda t: t.permute(*dims))

    def local(self) -> torch.Tensor:
        return TensorTransportRuntime.require().get(self.refs)

    def retain_grad(self) -> "TensorMeta":
        self.retain_grad_flag = True
        return self


class TensorStore:
    """Thread-safe refcounted tensor table; the single owner of rollout payloads on a worker."""

    def __init__(self, worker_id: int):
        self.worker_id = worker_id
        self._lock = threading.Lock()
        self._next = itertools.count(1)
        self._data: Dict[int, torch.Tensor] = {}
        self._refcnt: Dict[int, int] = {}

    def put(self, t: torch.Tensor) -> TensorRef:
        t = t.detach()
        if not t.is_contiguous():
            t = t.contiguous()
        with self._lock:
            key = next(self._next)
            self._data[key] = t
            self._refcnt[key] = 1
        return TensorRef(self.worker_id, key, tuple(t.shape), t.dtype, str(t.device))

    def get(self, key: int) -> torch.Tensor:
        with self._lock:
            try:
                return self._data[key]
            except KeyError:
                raise KeyError(f"worker {self.worker_id}: tensor key {key} is not (or no longer) stored") from None

    def incref(self, key: int) -> None:
        with self._lock:
            self._refcnt[key] += 1

    def decref(self, key: int) -> None:
        with self._lock:
            n = self._refcnt.get(key, 0) - 1
            if n <= 0:
                self._refcnt.pop(key, None)
                self._data.pop(key, None)
            else:
                self._refcnt[key] = n

    def clear(self) -> None:
        with self._lock:
            self._data.clear()
            self._refcnt.clear()

    def __len__(self) -> int:
        return len(self._data)

    def nbytes(self) -> int:
        with self._lock:
            return sum(t.numel() * t.element_size() for t in self._data.values())


class TransportSession:
    """Tracks refs created inside a ``with transport.session()`` block and frees them on exit."""

    def __init__(self, transport: "TensorTransport"):
        self.transport = transport
        self.created: List[TensorRef] = []

    def track(self, ref: TensorRef) -> TensorRef:
        self.created.append(ref)
        return ref

    def release(self) -> None:
        for r in self.created:
            self.transport.free(r)
        self.created.clear()


class TensorTransport(abc.ABC):
    """Backend-agnostic contract."""

    @abc.abstractmethod
    def put(self, tensor: torch.Tensor) -> TensorRef: ...

    @abc.abstractmethod
    def get(self, refs: Sequence[TensorRef]) -> torch.Tensor:
        """Materialise the rows of ``refs`` (concatenated along dim 0) on this process."""

    @abc.abstractmethod
    def free(self, ref: TensorRef) -> None: ...

    def is_ref(self, obj: Any) -> bool:
        return isinstance(obj, TensorRef)

    # ---- batched + tree helpers -------------------------------------------------------------
    def put_batch(self, tensors: Dict[str, torch.Tensor]) -> Dict[str, TensorMeta]:
        return {k: TensorMeta.from_refs([self.put(t)]) if t.dim() else self._put_scalar(t) for k, t in tensors.items()}

    def _put_scalar(self, t: torch.Tensor) -> TensorMeta:
        ref = self.put(t)
        return TensorMeta(refs=[ref], sizes=[1], shape=(), dtype=t.dtype, device=str(t.device))

    def get_batch(self, metas: Dict[str, TensorMeta]) -> Dict[str, torch.Tensor]:
        return {k: self.get(m.refs) for k, m in metas.items()}

    def dehydrate(self, tree: Any) -> Any:
        """Replace every tensor leaf by a handle (tree edited in place where mutable)."""
        return map_leaves(tree, torch.Tensor, lambda t: self._put_scalar(t) if t.dim() == 0 else TensorMeta.from_refs([self.put(t)]))

    def hydrate(self, tree: Any) -> Any:
        return map_leaves(tree, TensorMeta, lambda m: self.get(m.refs))

    def transform(self, meta: TensorMeta, fn: Callable[[torch.Tensor], torch.Tensor]) -> TensorMeta:
        return TensorMeta.from_refs([self.put(fn(self.get(meta.refs)))])

    def end_call(self) -> None:
        """Hook run after each role method (release borrowed views etc.)."""

    @contextlib.contextmanager
    def session(self) -> Iterator[TransportSession]:
        s = TransportSession(self)
        try:
            yield s
        finally:
            s.release()


REMOTE_OPS = frozenset({"incref", "decref", "send", "recv", "send_many", "recv_many", "get_cpu", "tensor_op", "stats", "clear"})


class WorkerLocalTransport(TensorTransport):
    """Store-backed transport living inside a worker process.

    ``send``/``recv`` move one stored tensor between two workers through the pool-wide process
    group (NCCL for CUDA tensors over NVLink, gloo for CPU tensors).
    """

    def __init__(self, worker_id: int, device: torch.device, comm: Optional[Any] = None):
        self.worker_id = worker_id
        self.device = torch.device(device)
        self.store = TensorStore(worker_id)
        self.comm = comm  # object with send(tensor, dst) / recv(tensor, src) (see group.comm)

    # ---- TensorTransport ---------------------------------------------------------------------
    def put(self, tensor: torch.Tensor) -> TensorRef:
        return self.store.put(tensor)

    def get(self, refs: Sequence[TensorRef]) -> torch.Tensor:
        parts = []
        for r in refs:
            if r.owner != self.worker_id:
                raise RuntimeError(f"worker {self.worker_id}: ref {r.key} is owned by worker {r.owner}; localize it first")
            parts.append(self._resolve(r))
        if len(parts) == 1:
            return parts[0]
        if parts and parts[0].dim() == 0:
            return torch.stack(parts)
        return torch.cat(parts, 0)

    def _resolve(self, ref: TensorRef) -> torch.Tensor:
        t = self.store.get(ref.key)
        if t.dim() and ref.shape and (ref.lo or ref.rows != t.shape[0]):
            t = t[ref.lo : ref.lo + ref.rows]
        return t

    def free(self, ref: TensorRef) -> None:
        if ref.owner == self.worker_id and ref.base is None:
            self.store.decref(ref.key)

    # ---- remote ops (invoked by the controller through Worker.transport_op) -------------------
    def incref(self, ref: TensorRef) -> None:
        self.store.incref(ref.key)

    def decref(self, ref: TensorRef) -> None:
        self.store.decref(ref.key)

    def send(self, ref: TensorRef, dst: int) -> None:
        self.comm.send(self._resolve(ref).contiguous(), dst)

    def recv(self, ref: TensorRef, src: int) -> TensorRef:
        dev = self.device if ref.device.startswith("cuda") else torch.device("cpu")
        buf = torch.empty(ref.shape, dtype=ref.dtype, device=dev)
        self.comm.recv(buf, src)
        return self.store.put(buf)

    # Several refs between the same two workers travel as ONE message per (dtype, device kind): the rows are packed into a flat buffer on
    # the sender and handed out as views of the received buffer (one NCCL / gloo launch per pair instead of one per tensor).
    @staticmethod
    def _pack_groups(refs: Sequence[TensorRef]) -> List[Tuple[Tuple[torch.dtype, bool], List[int]]]:
        groups: Dict[Tuple[torch.dtype, bool], List[int]] = {}
        for i, r in enumerate(refs):
            groups.setdefault((r.dtype, r.device.startswith("cuda")), []).append(i)
        return list(groups.items())

    def send_many(self, refs: Sequence[TensorRef], dst: int) -> int:
        """Returns the number of messages sent."""
        n = 0
        for _key, idx in self._pack_groups(refs):
            parts = [self._resolve(refs[i]).contiguous().reshape(-1) for i in idx]
            self.comm.send(parts[0] if len(parts) == 1 else torch.cat(parts), dst)
            n += 1
        self.messages_sent = getattr(self, "messages_sent", 0) + n
        return n

    def recv_many(self, refs: Sequence[TensorRef], src: int) -> List[TensorRef]:
        out: List[Optional[TensorRef]] = [None] * len(refs)
        for (dtype, on_cuda), idx in self._pack_groups(refs):
            sizes = [int(torch.Size(refs[i].shape).numel()) for i in idx]
            buf = torch.empty(sum(sizes), dtype=dtype, device=self.device if on_cuda else torch.device("cpu"))
            self.comm.recv(buf, src)
            off = 0
            for i, n in zip(idx, sizes):
                out[i] = self.store.put(buf[off : off + n].view(refs[i].shape))
                off += n
        return out  # type: ignore[return-value]

    def get_cpu(self, ref: TensorRef) -> torch.Tensor:
        return self._resolve(ref).detach().cpu()

    def tensor_op(self, ref: TensorRef, op: str, *args: Any) -> TensorRef:
        t = self._resolve(ref)
        if op == "getitem":
            out = t[args[0]]
        elif op == "reshape":
            out = t.reshape(args[0])
        elif op == "permute":
            out = t.permute(args[0])
        else:
            raise ValueError(f"unknown tensor op {op!r}")
        return self.store.put(out)

    def stats(self) -> Dict[str, int]:
        return {"tensors": len(self.store), "bytes": self.store.nbytes(), "messages_sent": getattr(self, "messages_sent", 0)}

    def clear(self) -> None:
        self.store.clear()

    def remote_op(self, op: str, *args: Any) -> Any:
        if op not in REMOTE_OPS:
            raise PermissionError(f"transport op {op!r} is not on the allow-list")
        return getattr(self, op)(*args)


def plan_localize(per_worker_payloads: Sequence[Any], worker_ids: Sequence[int]) -> List[Tuple[int, int, TensorRef]]:
    """List the ``(src, dst, ref)`` hops needed so that payload ``i`` only holds refs owned by ``worker_ids[i]``."""
    from unirl_b200.distributed.utils import iter_leaves

    hops: List[Tuple[int, int, TensorRef]] = []
    seen = set()
    for payload, dst in zip(per_worker_payloads, worker_ids):
        for _path, meta, _set in iter_leaves(payload, TensorMeta):
            for r in meta.refs:
                if isinstance(r, TensorRef) and r.owner != dst and (*r.ident, dst) not in seen:
                    seen.add((*r.ident, dst))
                    hops.append((r.owner, dst, r))
    return hops


def rewrite_refs(payload: Any, mapping: Dict[Tuple[int, int, int], TensorRef], dst: int) -> Any:
    """Substitute foreign refs in ``payload`` by their localized copies on ``dst``."""

    def fix(meta: TensorMeta) -> TensorMeta:
        new = [mapping.get((*r.ident, dst), r) if isinstance(r, TensorRef) else r for r in meta.refs]
        out = meta._with_refs(new, meta.sizes)
        out.grad, out.retain_grad_flag = meta.grad, meta.retain_grad_flag
        if new:
            out.device = new[0].device
        return out

    return map_leaves(payload, TensorMeta, fix)


__all__ = [
    "TensorRef",
    "TensorMeta",
    "TensorStore",
    "TensorTransport",
    "TensorTransportRuntime",
    "TransportSession",
    "WorkerLocalTransport",
    "REMOTE_OPS",
    "plan_localize",
    "rewrite_refs",
]
