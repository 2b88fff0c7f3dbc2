"""``Batch`` — dataclass containers whose fields know how they behave along the sample axis.

Every rollout / training payload in the framework (requests, tracks, segments, conditions)
is a ``@dataclass`` deriving from :class:`Batch`. Each field declares a *kind*:

* ``CONCAT``  – one row per sample (tensor dim 0, list element, nested ``Batch``, dict of those)
* ``PACKED``  – ragged per-sample data flattened along dim 0; the per-sample extents live in
  one hidden ``cu_seqlens`` vector per instance (exactly what varlen attention kernels take)
* ``SHARED``  – identical for all samples (schedules, configs)
* ``MAX`` / ``MIN`` / ``SUM`` / ``MEAN`` – per-instance scalars folded on concat

and the base class derives ``concat / chunk / select / slice / repeat_interleave / to_device /
clone / map`` from that declaration.

Design: instead of one hand-written walker per operation, every sample-axis operation is an
``_AxisOp`` object with four leaf rules (tensor, sequence, nested batch, packed tensor) and one
generic tree walker applies it.  Behavioural parity target: ``unirl/distributed/tensor/batch.py``
(field kinds ``:85-95``, field constructors ``:107-197``, ``Batch`` ``:551-900``).
"""

from __future__ import annotations

import copy
import dataclasses
import inspect
import uuid
from enum import Enum, auto
from typing import Any, Callable, Dict, List, Optional, Sequence, Type, TypeVar, Union

import torch

B = TypeVar("B", bound="Batch")

_KIND = "kind"
_CU_ATTR = "_packed_cu_seqlens"


class FieldKind(Enum):
    CONCAT = auto()
    SHARED = auto()
    MAX = auto()
    MIN = auto()
    SUM = auto()
    MEAN = auto()
    PACKED = auto()


_FOLD_KINDS = (FieldKind.MAX, FieldKind.MIN, FieldKind.SUM, FieldKind.MEAN)
_DC_PARAMS = frozenset(inspect.signature(dataclasses.field).parameters)


# --------------------------------------------------------------------------- field constructors
def field(**kw: Any) -> Any:
    """``dataclasses.field`` with open metadata: unknown kwargs (``kind=…``) land in ``metadata``."""
    meta = dict(kw.pop("metadata", None) or {})
    passthrough = {}
    for key, val in kw.items():
        (passthrough if key in _DC_PARAMS else meta)[key] = val
    return dataclasses.field(metadata=meta, **passthrough)


def _kinded(kind: FieldKind) -> Callable[..., Any]:
    def ctor(**kw: Any) -> Any:
        return field(kind=kind, **kw)

    ctor.__name__ = f"{kind.name.lower()}_field"
    ctor.__doc__ = f"Declare a {kind.name} field (see module docstring)."
    return ctor


concat_field = _kinded(FieldKind.CONCAT)
packed_field = _kinded(FieldKind.PACKED)
shared_field = _kinded(FieldKind.SHARED)
max_field = _kinded(FieldKind.MAX)
min_field = _kinded(FieldKind.MIN)
sum_field = _kinded(FieldKind.SUM)
mean_field = _kinded(FieldKind.MEAN)


def kind_of(f: dataclasses.Field) -> FieldKind:
    return f.metadata.get(_KIND, FieldKind.SHARED)


# --------------------------------------------------------------------------- leaf helpers
def leading_size(value: Any) -> Optional[int]:
    """Sample-axis extent of a value, ``None`` when it has none."""
    if isinstance(value, torch.Tensor):
        return int(value.shape[0]) if value.dim() else None
    if isinstance(value, (list, tuple)):
        return len(value)
    if isinstance(value, Batch):
        return value.batch_size
    if isinstance(value, dict):
        for v in value.values():
            n = leading_size(v)
            if n is not None:
                return n
    return None


def _fold(values: List[Any], kind: FieldKind) -> Any:
    vals = [v for v in values if v is not None]
    if not vals:
        return None
    if all(isinstance(v, torch.Tensor) for v in vals):
        s = torch.stack(vals)
        return {FieldKind.MAX: s.amax, FieldKind.MIN: s.amin, FieldKind.SUM: s.sum, FieldKind.MEAN: s.mean}[kind](dim=0)
    if kind is FieldKind.MAX:
        return max(vals)
    if kind is FieldKind.MIN:
        return min(vals)
    total = sum(vals)
    return total if kind is FieldKind.SUM else total / len(vals)


class _AxisOp:
    """A unary operation along the sample axis, applied leaf-wise by :func:`_walk`."""

    def tensor(self, t: torch.Tensor) -> torch.Tensor:  # batched tensor [n, ...]
        raise NotImplementedError

    def seq(self, s: Union[list, tuple]) -> Union[list, tuple]:  # len == n
        raise NotImplementedError

    def batch(self, b: "Batch") -> "Batch":
        raise NotImplementedError

    def packed(self, data: torch.Tensor, cu: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def cu(self, cu: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


def _walk(op: _AxisOp, value: Any, n: int) -> Any:
    if value is None:
        return None
    if isinstance(value, torch.Tensor):
        return op.tensor(value) if value.dim() and int(value.shape[0]) == n else value
    if isinstance(value, (list, tuple)):
        return op.seq(value) if len(value) == n else value
    if isinstance(value, dict):
        return {k: _walk(op, v, n) for k, v in value.items()}
    if isinstance(value, Batch):
        return op.batch(value)
    return value


def _lens(cu: torch.Tensor) -> torch.Tensor:
    return cu[1:] - cu[:-1]


def _cu_from_lens(lens: torch.Tensor) -> torch.Tensor:
    out = torch.zeros(lens.numel() + 1, dtype=torch.long, device=lens.device)
    if lens.numel():
        out[1:] = torch.cumsum(lens.to(torch.long), 0)
    return out


def _gather_rows(data: torch.Tensor, cu: torch.Tensor, order: Sequence[int]) -> torch.Tensor:
    """Concatenate the ragged rows ``order`` of a packed tensor with one index_select."""
    if not len(order):
        return data[:0]
    cu_l = cu.tolist()
    idx = torch.cat([torch.arange(cu_l[i], cu_l[i + 1]) for i in order])
    return data.index_select(0, idx.to(data.device))


class _Select(_AxisOp):
    def __init__(self, indices: Union[torch.Tensor, Sequence[int]]):
        self.idx_t = indices if isinstance(indices, torch.Tensor) else torch.tensor(list(indices), dtype=torch.long)
        self.idx_l = [int(i) for i in self.idx_t.tolist()]

    def tensor(self, t):
        return t.index_select(0, self.idx_t.to(t.device))

    def seq(self, s):
        return type(s)(s[i] for i in self.idx_l)

    def batch(self, b):
        return b.select(self.idx_t)

    def packed(self, data, cu):
        return _gather_rows(data, cu, self.idx_l)

    def cu(self, cu):
        return _cu_from_lens(_lens(cu)[self.idx_t.to(cu.device)])


class _Slice(_AxisOp):
    def __init__(self, lo: int, hi: int):
        self.lo, self.hi = lo, hi

    def tensor(self, t):
        return t[self.lo : self.hi]

    def seq(self, s):
        return s[self.lo : self.hi]

    def batch(self, b):
        return b.slice(self.lo, self.hi)

    def packed(self, data, cu):
        return data[int(cu[self.lo]) : int(cu[self.hi])]

    def cu(self, cu):
        return cu[self.lo : self.hi + 1] - cu[self.lo]


class _Repeat(_AxisOp):
    def __init__(self, n: int):
        self.n = n

    def tensor(self, t):
        return t.repeat_interleave(self.n, dim=0)

    def seq(self, s):
        return type(s)(copy.copy(x) for x in s for _ in range(self.n))

    def batch(self, b):
        return b.repeat_interleave(self.n)

    def packed(self, data, cu):
        rows = [i for i in range(cu.numel() - 1) for _ in range(self.n)]
        return _gather_rows(data, cu, rows)

    def cu(self, cu):
        return _cu_from_lens(_lens(cu).repeat_interleave(self.n))


def _join(values: List[Any], sizes: List[int]) -> Any:
    """Concatenate per-instance CONCAT values (the n-ary counterpart of an ``_AxisOp``)."""
    live = [(v, n) for v, n in zip(values, sizes) if v is not None]
    if not live:
        return None
    vals = [v for v, _ in live]
    head = vals[0]
    if all(isinstance(v, torch.Tensor) for v in vals):
        aligned = [v.dim() > 0 and int(v.shape[0]) == n for v, n in live]
        if all(aligned):
            return torch.cat(vals, 0)
        if not any(aligned):
            return head
        raise ValueError("concat field mixes batched and unbatched tensors")
    if all(isinstance(v, (list, tuple)) for v in vals) and all(len(v) == n for v, n in live):
        flat = [x for v in vals for x in v]
        return flat if isinstance(head, list) else tuple(flat)
    if all(isinstance(v, dict) for v in vals):
        keys = sorted({k for v in vals for k in v})
        return {k: _join([v.get(k) if isinstance(v, dict) else None for v in values], sizes) for k in keys}
    if all(isinstance(v, Batch) for v in vals):
        return type(head).concat(vals)
    # replicated payload: accept only when every instance agrees
    if isinstance(head, torch.Tensor):
        if all(isinstance(v, torch.Tensor) and v.shape == head.shape and torch.equal(v.to(head.device), head) for v in vals[1:]):
            return head
    elif all(v == head for v in vals[1:]):
        return copy.deepcopy(head)
    raise ValueError(f"cannot concat {[type(v).__name__ for v in values]} with batch sizes {sizes}")


def _tree_apply(value: Any, fn: Callable[[torch.Tensor], torch.Tensor]) -> Any:
    if isinstance(value, torch.Tensor):
        return fn(value)
    if isinstance(value, Batch):
        return value._tensor_map(fn)
    if isinstance(value, dict):
        return {k: _tree_apply(v, fn) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_tree_apply(v, fn) for v in value)
    return value


# --------------------------------------------------------------------------- Batch
class Batch:
    """Base for field-kind aware dataclass containers (see module docstring)."""

    # ---- hidden state ------------------------------------------------------------------
    @property
    def _eid(self) -> str:
        eid = self.__dict__.get("_eid_cache")
        if eid is None:
            eid = uuid.uuid4().hex
            object.__setattr__(self, "_eid_cache", eid)
        return eid

    @property
    def cu_seqlens(self) -> Optional[torch.Tensor]:
        """``[N+1]`` cumulative offsets shared by all PACKED fields (``None`` if unset)."""
        return self.__dict__.get(_CU_ATTR)

    def _set_cu(self, cu: Optional[torch.Tensor]) -> None:
        object.__setattr__(self, _CU_ATTR, cu)

    @property
    def lengths(self) -> Optional[torch.Tensor]:
        cu = self.cu_seqlens
        return None if cu is None else _lens(cu)

    @classmethod
    def _fields(cls) -> Sequence[dataclasses.Field]:
        return dataclasses.fields(cls)  # type: ignore[arg-type]

    @property
    def batch_size(self) -> int:
        cu = self.cu_seqlens
        if cu is not None:
            return int(cu.numel()) - 1
        for f in self._fields():
            if kind_of(f) is FieldKind.CONCAT:
                n = leading_size(getattr(self, f.name))
                if n is not None:
                    return n
        return 0

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def pack(cls: Type[B], **kw: Any) -> B:
        """Build an instance, flattening per-sample tensor lists given for PACKED fields.

        All packed fields of one instance must agree on the per-sample extents.
        """
        packed_names = {f.name for f in cls._fields() if kind_of(f) is FieldKind.PACKED}
        cu: Optional[torch.Tensor] = None
        for name in packed_names & kw.keys():
            rows = kw[name]
            if rows is None or isinstance(rows, torch.Tensor):
                continue
            rows = list(rows)
            lens = torch.tensor([int(r.shape[0]) for r in rows], dtype=torch.long)
            this_cu = _cu_from_lens(lens)
            if cu is None:
                cu = this_cu
            elif not torch.equal(cu, this_cu):
                raise ValueError(f"{cls.__name__}.pack: field {name!r} disagrees on per-sample sizes")
            kw[name] = torch.cat(rows, 0) if rows else torch.zeros(0)
        obj = cls(**kw)
        if cu is not None:
            obj._set_cu(cu)
        return obj

    def _rebuild(self: B, values: Dict[str, Any], cu: Any = "keep") -> B:
        """Same-type reconstruction from field values, carrying the hidden offsets."""
        out = type(self)(**values)
        out._set_cu(self.cu_seqlens if isinstance(cu, str) else cu)
        return out

    def _values(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in self._fields()}

    # ---- n-ary -----------------------------------------------------------------------------
    @classmethod
    def concat(cls: Type[B], items: Sequence[B]) -> B:
        items = list(items)
        if not items:
            raise ValueError(f"{cls.__name__}.concat: nothing to concatenate")
        if len(items) == 1:
            return items[0]
        sizes = [it.batch_size for it in items]
        out: Dict[str, Any] = {}
        for f in cls._fields():
            kind = kind_of(f)
            vals = [getattr(it, f.name) for it in items]
            if kind is FieldKind.CONCAT:
                out[f.name] = _join(vals, sizes)
            elif kind is FieldKind.PACKED:
                live = [v for v in vals if v is not None]
                if live and isinstance(live[0], Batch):  # tensor handles: join the handle lists, rows stay where they are
                    out[f.name] = type(live[0]).concat(live)
                else:
                    out[f.name] = torch.cat(live, 0) if live else None
            elif kind in _FOLD_KINDS:
                out[f.name] = _fold(vals, kind)
            else:
                out[f.name] = next((v for v in vals if v is not None), None)
        cus = [it.cu_seqlens for it in items]
        cu = None
        if any(c is not None for c in cus):
            if any(c is None for c in cus):
                raise ValueError(f"{cls.__name__}.concat: some instances lack cu_seqlens")
            cu = _cu_from_lens(torch.cat([_lens(c) for c in cus]))
        return items[0]._rebuild(out, cu)

    def concat_with(self: B, *others: B) -> B:
        return type(self).concat([self, *others])

    # ---- unary axis ops ------------------------------------------------------------------
    def _axis(self: B, op: _AxisOp) -> B:
        n = self.batch_size
        cu = self.cu_seqlens
        out: Dict[str, Any] = {}
        for f in self._fields():
            kind, val = kind_of(f), getattr(self, f.name)
            if kind is FieldKind.CONCAT:
                out[f.name] = _walk(op, val, n)
            elif kind is FieldKind.PACKED and val is not None:
                if cu is None:
                    raise ValueError(f"{type(self).__name__}.{f.name}: packed field without cu_seqlens")
                out[f.name] = op.packed(val, cu)
            else:
                out[f.name] = val
        return self._rebuild(out, None if cu is None else op.cu(cu))

    def select(self: B, indices: Union[torch.Tensor, Sequence[int]]) -> B:
        return self._axis(_Select(indices))

    def slice(self: B, start: int, end: int) -> B:
        return self._axis(_Slice(int(start), int(end)))

    def repeat_interleave(self: B, n: int) -> B:
        """Each sample ``n`` times, siblings adjacent (``[s0,s0,…,s1,s1,…]``)."""
        if n < 1:
            raise ValueError("repeat_interleave: n must be >= 1")
        return self if n == 1 else self._axis(_Repeat(int(n)))

    def chunk(self: B, n: int) -> List[B]:
        total = self.batch_size
        if n < 1 or total % n:
            raise ValueError(f"{type(self).__name__}.chunk: batch_size={total} not divisible by {n}")
        step = total // n
        return [self.slice(i * step, (i + 1) * step) for i in range(n)]

    def __len__(self) -> int:
        return self.batch_size

    # ---- whole-tree ops --------------------------------------------------------------------
    def _tensor_map(self: B, fn: Callable[[torch.Tensor], torch.Tensor]) -> B:
        out = {k: _tree_apply(v, fn) for k, v in self._values().items()}
        cu = self.cu_seqlens
        return self._rebuild(out, cu)

    def to_device(self: B, device: Union[str, torch.device]) -> B:
        return self._tensor_map(lambda t: t.to(device))

    to = to_device

    def clone(self: B) -> B:
        def dup(v: Any) -> Any:
            if isinstance(v, torch.Tensor):
                return v.clone()
            if isinstance(v, Batch):
                return v.clone()
            if isinstance(v, dict):
                return {k: dup(x) for k, x in v.items()}
            if isinstance(v, (list, tuple)):
                return type(v)(dup(x) for x in v)
            return copy.deepcopy(v)

        cu = self.cu_seqlens
        return self._rebuild({k: dup(v) for k, v in self._values().items()}, None if cu is None else cu.clone())

    def map(self: B, fn: Callable[[Any], Any]) -> B:
        """Apply ``fn`` to each top-level field value; hidden offsets are kept."""
        return self._rebuild({k: fn(v) for k, v in self._values().items()})

    def replace(self: B, **changes: Any) -> B:
        vals = self._values()
        vals.update(changes)
        return self._rebuild(vals)


__all__ = [
    "Batch",
    "FieldKind",
    "field",
    "concat_field",
    "packed_field",
    "shared_field",
    "max_field",
    "min_field",
    "sum_field",
    "mean_field",
    "kind_of",
    "leading_size",
]
