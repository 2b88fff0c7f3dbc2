"""Aggregation helpers for logged metrics.  Parity: ``unirl/utils/wandb_metrics.py``."""

from __future__ import annotations

from typing import Any, Dict, Iterable, List

import torch


def tensor_stats(t: torch.Tensor, prefix: str) -> Dict[str, float]:
    t = t.float().flatten()
    if not t.numel():
        return {}
    return {f"{prefix}_mean": float(t.mean()), f"{prefix}_std": float(t.std()) if t.numel() > 1 else 0.0,
            f"{prefix}_min": float(t.min()), f"{prefix}_max": float(t.max())}


def flatten_metrics(metrics: Dict[str, Any], prefix: str = "") -> Dict[str, float]:
    out: Dict[str, float] = {}
    for k, v in metrics.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            out.update(flatten_metrics(v, key + "/"))
        elif isinstance(v, (list, tuple)) and v and all(isinstance(x, (int, float)) for x in v):
            out[key] = sum(v) / len(v)
        elif isinstance(v, torch.Tensor) and v.numel() == 1:
            out[key] = float(v)
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            out[key] = float(v)
    return out


def mean_of_dicts(items: Iterable[Dict[str, float]]) -> Dict[str, float]:
    items = list(items)
    keys = {k for d in items for k in d}
    return {k: sum(d[k] for d in items if k in d) / sum(1 for d in items if k in d) for k in keys}


__all__ = ["tensor_stats", "flatten_metrics", "mean_of_dicts"]
