"""Reward → advantage normalisers over explicit index groups (ragged groups allowed).

``normalize_grouped``: per-group mean; divisor = group Bessel std + ε, or the batch-wide std when
``use_global_std``; optional symmetric outlier trimming for the statistics and a final clip.
Parity: ``unirl/algorithms/normalizers.py:8-136``.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch


def normalize_grouped(rewards: torch.Tensor, group_indices: List[List[int]], epsilon: float = 1e-8, clip_max: Optional[float] = None,
                      trim_outliers_ratio: float = 0.0, use_global_std: bool = False) -> torch.Tensor:
    adv = torch.zeros_like(rewards)
    batch_std = rewards.std() + epsilon if use_global_std else None
    for rows in group_indices:
        if not rows:
            continue
        g = rewards[rows]
        stats = g
        if trim_outliers_ratio > 0 and len(rows) > 2:
            k = int(len(rows) * trim_outliers_ratio)
            if k > 0 and 2 * k < len(rows):
                stats = torch.sort(g).values[k:-k]
        std = batch_std if use_global_std else stats.std() + epsilon
        adv[rows] = (g - stats.mean()) / std
    return adv.clamp(-clip_max, clip_max) if clip_max is not None else adv


def normalize_global(rewards: torch.Tensor, epsilon: float = 1e-8, clip_max: Optional[float] = None) -> torch.Tensor:
    adv = (rewards - rewards.mean()) / (rewards.std() + epsilon)
    return adv.clamp(-clip_max, clip_max) if clip_max is not None else adv


def _clean_gid(gid: Any) -> Optional[str]:
    if gid is None:
        return None
    s = str(gid).strip()
    return s or None


def require_valid_group_ids(group_ids: List[str]) -> List[str]:
    out = []
    for i, g in enumerate(group_ids):
        c = _clean_gid(g)
        if c is None:
            raise ValueError(f"adv_normalization_scope='group' needs a non-empty group_id for every sample (sample {i})")
        out.append(c)
    return out


def build_group_index_map(group_ids: List[str]) -> Dict[str, List[int]]:
    groups: Dict[str, List[int]] = {}
    for i, g in enumerate(group_ids):
        c = _clean_gid(g)
        if c is not None:
            groups.setdefault(c, []).append(i)
    return groups


def require_expected_group_sizes(group_index_map: Dict[str, List[int]], samples_per_prompt: int) -> List[List[int]]:
    want = max(1, int(samples_per_prompt))
    bad = [(g, len(ix)) for g, ix in group_index_map.items() if len(ix) != want]
    if bad:
        shown = ", ".join(f"{g!r}:{n}" for g, n in bad[:5]) + (", ..." if len(bad) > 5 else "")
        raise ValueError(f"every group must hold samples_per_prompt={want} samples; offending groups: {shown}")
    return list(group_index_map.values())


__all__ = ["normalize_grouped", "normalize_global", "require_valid_group_ids", "build_group_index_map", "require_expected_group_sizes"]
