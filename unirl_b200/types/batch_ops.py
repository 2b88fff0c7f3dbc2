"""Free-function batch utilities over loose value trees (dict / list / tensor / ``Batch``).

Parity: ``unirl/types/batch_ops.py`` (``copy_mapping``, ``batch_clone``, ``batch_move``,
``batch_slice``, ``batch_pad``, ``batch_concat``, ``batch_reindex``).
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Sequence, Union

import torch
import torch.nn.functional as F

from unirl_b200.distributed.tensor.batch import Batch, _join, _tree_apply


def copy_mapping(mapping: Optional[Mapping[str, Any]]) -> Dict[str, Any]:
    return dict(mapping) if mapping else {}


def batch_clone(value: Any) -> Any:
    if isinstance(value, Batch):
        return value.clone()
    return _tree_apply(value, lambda t: t.clone())


def batch_move(value: Any, device: Union[str, torch.device]) -> Any:
    return _tree_apply(value, lambda t: t.to(device))


def batch_slice(value: Any, start: int, end: int, batch_size: Optional[int] = None) -> Any:
    if isinstance(value, Batch):
        return value.slice(start, end)
    if isinstance(value, torch.Tensor):
        ok = value.dim() > 0 and (batch_size is None or value.shape[0] == batch_size)
        return value[start:end] if ok else value
    if isinstance(value, (list, tuple)):
        return value[start:end] if batch_size is None or len(value) == batch_size else value
    if isinstance(value, dict):
        return {k: batch_slice(v, start, end, batch_size) for k, v in value.items()}
    return value


def batch_pad(t: torch.Tensor, target_len: int, dim: int = 1, value: float = 0.0) -> torch.Tensor:
    gap = target_len - t.shape[dim]
    if gap < 0:
        raise ValueError(f"batch_pad: length {t.shape[dim]} exceeds target {target_len}")
    if gap == 0:
        return t
    spec = [0, 0] * (t.dim() - 1 - dim) + [0, gap]
    return F.pad(t, spec, value=value)


def batch_concat(values: Sequence[Any], batch_sizes: Optional[Sequence[int]] = None) -> Any:
    values = list(values)
    if batch_sizes is None:
        from unirl_b200.distributed.tensor.batch import leading_size

        batch_sizes = [leading_size(v) or 0 for v in values]
    return _join(values, list(batch_sizes))


def batch_reindex(value: Any, indices: Union[torch.Tensor, Sequence[int]], batch_size: Optional[int] = None) -> Any:
    idx = indices if isinstance(indices, torch.Tensor) else torch.tensor(list(indices), dtype=torch.long)
    if isinstance(value, Batch):
        return value.select(idx)
    if isinstance(value, torch.Tensor):
        ok = value.dim() > 0 and (batch_size is None or value.shape[0] == batch_size)
        return value.index_select(0, idx.to(value.device)) if ok else value
    if isinstance(value, (list, tuple)):
        return type(value)(value[int(i)] for i in idx.tolist()) if batch_size is None or len(value) == batch_size else value
    if isinstance(value, dict):
        return {k: batch_reindex(v, idx, batch_size) for k, v in value.items()}
    return value


__all__ = ["copy_mapping", "batch_clone", "batch_move", "batch_slice", "batch_pad", "batch_concat", "batch_reindex"]
