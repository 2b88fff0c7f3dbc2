"""Sample-axis split / merge of arbitrary call payloads (used by DP dispatch and collect).

Parity: ``unirl/distributed/tensor/pytree.py:34-95`` (``infer_batch_size``), ``:98-193``
(``pytree_chunk``), ``:196-246`` (``pytree_cat``).
"""

from __future__ import annotations

from typing import Any, List, Optional

import numpy as np
import torch

from unirl_b200.distributed.tensor.batch import Batch
from unirl_b200.distributed.tensor.transport import TensorMeta
from unirl_b200.distributed.utils import Broadcast


def _axis_size(v: Any) -> Optional[int]:
    if isinstance(v, Broadcast):
        return None
    if isinstance(v, TensorMeta):
        return int(v.shape[0]) if v.shape else None
    if isinstance(v, (torch.Tensor, np.ndarray)):
        return int(v.shape[0]) if v.ndim else None
    if isinstance(v, list):
        return len(v)
    if isinstance(v, Batch):
        return v.batch_size or None
    if isinstance(v, tuple):
        children = v
    elif isinstance(v, dict):
        children = v.values()
    else:
        return None
    for c in children:
        n = _axis_size(c)
        if n is not None:
            return n
    return None


def infer_batch_size(args: tuple, kwargs: dict) -> Optional[int]:
    """First sample-axis extent found in ``args`` then ``kwargs`` (``None`` ⇒ pure broadcast call)."""
    return _axis_size((*args, *kwargs.values()))


def _even(batch_size: int, n: int) -> int:
    if batch_size % n:
        raise ValueError(f"batch_size={batch_size} not divisible by dp_size={n}")
    return batch_size // n


def pytree_chunk(value: Any, dp_size: int, batch_size: int) -> List[Any]:
    """Split ``value`` into ``dp_size`` shards along dim 0; anything not aligned to ``batch_size`` is replicated."""
    rep = lambda: [value] * dp_size  # noqa: E731
    if isinstance(value, Broadcast):
        return [value.value] * dp_size
    if isinstance(value, TensorMeta):
        if not value.shape or value.shape[0] != batch_size:
            return rep()
        _even(batch_size, dp_size)
        return value.chunk_refs(dp_size)
    if isinstance(value, (torch.Tensor, np.ndarray)):
        if not value.ndim or value.shape[0] != batch_size:
            return rep()
        step = _even(batch_size, dp_size)
        return [value[i * step : (i + 1) * step] for i in range(dp_size)]
    if isinstance(value, list):
        if len(value) != batch_size:
            return rep()
        step = _even(batch_size, dp_size)
        return [value[i * step : (i + 1) * step] for i in range(dp_size)]
    if isinstance(value, dict):
        cols = {k: pytree_chunk(v, dp_size, batch_size) for k, v in value.items()}
        return [{k: cols[k][i] for k in value} for i in range(dp_size)]
    if isinstance(value, tuple):
        cols = [pytree_chunk(v, dp_size, batch_size) for v in value]
        return [tuple(c[i] for c in cols) for i in range(dp_size)]
    if isinstance(value, Batch):
        return value.chunk(dp_size) if value.batch_size == batch_size else rep()
    return rep()


def pytree_cat(results: List[Any]) -> Any:
    """Merge same-structured per-shard results along dim 0."""
    if not results:
        return None
    head = results[0]
    if head is None:
        return None
    if isinstance(head, TensorMeta):
        return TensorMeta.concat(results)
    if isinstance(head, torch.Tensor):
        return torch.stack(results) if head.dim() == 0 else torch.cat(results, 0)
    if isinstance(head, np.ndarray):
        return np.concatenate(results, 0)
    if isinstance(head, list):
        return [x for r in results for x in r]
    if isinstance(head, tuple):
        return tuple(pytree_cat([r[i] for r in results]) for i in range(len(head)))
    if isinstance(head, dict):
        return {k: pytree_cat([r[k] for r in results]) for k in head}
    if isinstance(head, Batch):
        return type(head).concat(results)
    return head


__all__ = ["infer_batch_size", "pytree_chunk", "pytree_cat"]
