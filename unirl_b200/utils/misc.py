"""Seeding and small numeric helpers.  Parity: ``unirl/utils/misc.py`` (``set_seed`` ``:53-82``, ``aggregate_numeric_metrics``)."""

from __future__ import annotations

import os
import random
from typing import Any, Dict, Iterable, List, Mapping

import numpy as np
import torch


def set_seed(seed: int, deterministic: bool = False) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)


def aggregate_numeric_metrics(items: Iterable[Mapping[str, Any]]) -> Dict[str, Any]:
    """Mean of every numeric key over the dicts that carry it; non-numeric values keep the last one seen."""
    sums: Dict[str, float] = {}
    counts: Dict[str, int] = {}
    other: Dict[str, Any] = {}
    for d in items:
        for k, v in d.items():
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                if isinstance(v, torch.Tensor) and v.numel() == 1:
                    v = float(v)
                else:
                    other[k] = v
                    continue
            sums[k] = sums.get(k, 0.0) + float(v)
            counts[k] = counts.get(k, 0) + 1
    out: Dict[str, Any] = {k: sums[k] / counts[k] for k in sums}
    out.update({k: v for k, v in other.items() if k not in out})
    return out


__all__ = ["set_seed", "aggregate_numeric_metrics"]
