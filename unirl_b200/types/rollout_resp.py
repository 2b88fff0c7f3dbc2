"""``RolloutTrack`` / ``RolloutResp`` — rollout outputs with per-track lineage.

A response is a dict of tracks; each track is one modality at one lifecycle stage.  ``parent_ids``
define the GRPO groups (siblings share a parent and are adjacent), so group statistics are one
``view(n_groups, branch)`` away.  Parity: ``unirl/types/rollout_resp.py:71-333`` (track, advantages),
``:391-631`` (response, split, reward propagation).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Tuple, Type

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, max_field, shared_field
from unirl_b200.types.conditions.base import Condition
from unirl_b200.types.media_preview import MediaPreview
from unirl_b200.types.rollout_req import _fan_out
from unirl_b200.types.segments.base import Segment


def hydrate_if_handle(value: Any) -> Any:
    """Controller-side: turn a ``TensorMeta`` into a tensor (small fields like rewards only)."""
    from unirl_b200.distributed.tensor.transport import TensorMeta

    if isinstance(value, TensorMeta):
        return value.local() if value.refs else None
    return value


@dataclass
class RolloutTrack(Batch):
    sample_ids: List[str] = concat_field(default_factory=list)
    parent_ids: Optional[List[str]] = concat_field(default=None)
    parent_track: Optional[str] = shared_field(default=None)
    conditions: Dict[str, Condition] = concat_field(default_factory=dict)
    segment: Optional[Segment] = concat_field(default=None)
    decoded: Optional[Any] = concat_field(default=None)
    media_preview: Optional[MediaPreview] = shared_field(default=None)
    rewards: Optional[torch.Tensor] = concat_field(default=None)
    component_rewards: Optional[Dict[str, torch.Tensor]] = concat_field(default=None)
    advantages: Optional[torch.Tensor] = concat_field(default=None)
    status: Optional[torch.Tensor] = concat_field(default=None)

    @property
    def batch_size(self) -> int:
        return len(self.sample_ids) if self.sample_ids else super().batch_size

    @property
    def group_ids(self) -> List[str]:
        return list(self.parent_ids) if self.parent_ids is not None else list(self.sample_ids)

    def metadata_only(self) -> "RolloutTrack":
        light = copy.copy(self)
        light.conditions, light.segment, light.decoded = {}, None, None
        return light

    def split(self) -> List["RolloutTrack"]:
        gids = self.group_ids
        if not gids:
            return [self]
        rows: Dict[str, List[int]] = {}
        for i, g in enumerate(gids):
            rows.setdefault(g, []).append(i)
        return [self.select(torch.tensor(ix)) for ix in rows.values()]

    def fork_track(self, parent_name: str, child_name: str, branch: int,
                   decode_to_condition: Optional[Callable[["RolloutTrack"], Dict[str, Condition]]] = None,
                   new_segment: Optional[Segment] = None) -> "RolloutTrack":
        """Track → child track fan-out (``N`` → ``N·branch``), siblings adjacent."""
        if not self.sample_ids:
            raise ValueError("fork_track: track has no sample_ids")
        if branch < 1:
            raise ValueError(f"fork_track: branch must be >= 1, got {branch}")
        ids, parents = _fan_out(self.sample_ids, child_name[:1] or "c", branch)
        conds = {} if decode_to_condition is None else {k: c.repeat_interleave(branch) for k, c in decode_to_condition(self).items()}
        return RolloutTrack(sample_ids=ids, parent_ids=parents, parent_track=parent_name, conditions=conds, segment=new_segment)

    def compute_advantages(self, normalize: bool = True, eps: float = 1e-8, scope: str = "group",
                           use_global_std: bool = False) -> "RolloutTrack":
        """Group-relative advantages.

        ``scope="group"``: ``(r − mean_g) / sqrt(var_g + eps)`` with population variance (single-sample
        groups degrade to 0); ``use_global_std`` swaps the divisor for the batch-wide Bessel std
        ``+ eps``.  ``scope="global"``: ``(r − mean) / (std + eps)`` over the whole batch.
        """
        if self.rewards is None:
            raise ValueError("compute_advantages: track has no rewards")
        n = len(self.sample_ids)
        if n == 0:
            return self
        r = hydrate_if_handle(self.rewards).to(torch.float32)
        if scope == "global":
            adv = r - r.mean()
            return self.replace(advantages=adv / (r.std() + eps) if normalize else adv)
        if self.parent_ids is None:
            return self.replace(advantages=torch.zeros_like(r))
        groups = list(dict.fromkeys(self.parent_ids))
        if n % len(groups):
            raise ValueError(f"compute_advantages: {n} samples do not form {len(groups)} equal groups")
        branch = n // len(groups)
        if list(self.parent_ids) != [g for g in groups for _ in range(branch)]:
            raise ValueError("compute_advantages: siblings must be adjacent (group-by-parent order)")
        rg = r.view(len(groups), branch)
        adv = rg - rg.mean(1, keepdim=True)
        if normalize:
            adv = adv / ((r.std() + eps) if use_global_std else (rg.var(1, unbiased=False, keepdim=True) + eps).sqrt())
        return self.replace(advantages=adv.flatten())


def _root_groups(resp: "RolloutResp", name: str) -> List[str]:
    """Root-track group id of every sample of track ``name`` (walks ``parent_track`` upwards)."""
    t = resp.tracks[name]
    if t.parent_track is None:
        return t.group_ids
    if t.parent_ids is None:
        raise RuntimeError(f"track {name!r} has a parent_track but no parent_ids")
    up = _root_groups(resp, t.parent_track)
    row = {sid: i for i, sid in enumerate(resp.tracks[t.parent_track].sample_ids)}
    return [up[row[p]] for p in t.parent_ids]


@dataclass
class RolloutResp(Batch):
    tracks: Dict[str, RolloutTrack] = concat_field(default_factory=dict)
    reward_compute_s: float = max_field(default=0.0)

    def __post_init__(self) -> None:
        for name, t in self.tracks.items():
            if t.parent_ids is not None and len(t.parent_ids) != len(t.sample_ids):
                raise ValueError(f"track {name!r}: {len(t.parent_ids)} parent_ids for {len(t.sample_ids)} samples")
            if t.parent_track is None:
                continue
            if t.parent_track not in self.tracks:
                raise ValueError(f"track {name!r}: parent_track {t.parent_track!r} not in {sorted(self.tracks)}")
            if t.parent_ids is not None:
                known = set(self.tracks[t.parent_track].sample_ids)
                stray = [p for p in t.parent_ids if p not in known]
                if stray:
                    raise ValueError(f"track {name!r}: {len(stray)} parent ids unknown to {t.parent_track!r}, e.g. {stray[:3]}")

    @property
    def batch_size(self) -> int:
        return max((t.batch_size for t in self.tracks.values()), default=0)

    def metadata_only(self) -> "RolloutResp":
        return RolloutResp({k: t.metadata_only() for k, t in self.tracks.items()}, self.reward_compute_s)

    def root_track(self) -> RolloutTrack:
        roots = [k for k, t in self.tracks.items() if t.parent_track is None]
        if len(roots) != 1:
            raise RuntimeError(f"expected exactly one root track, found {sorted(roots)}")
        return self.tracks[roots[0]]

    def tracks_with_segment_types(self, segment_types: Iterable[Type[Segment]]) -> List[Tuple[str, RolloutTrack]]:
        want = set(segment_types)
        return [(k, t) for k, t in self.tracks.items() if t.segment is not None and type(t.segment) in want]

    def split(self) -> List["RolloutResp"]:
        """One response per root group, each carrying that group's whole subtree."""
        if not self.tracks:
            return [self]
        root_gids = self.root_track().group_ids
        if not root_gids:
            return [self]
        per_track = {k: _root_groups(self, k) for k in self.tracks}
        out = []
        for g in dict.fromkeys(root_gids):
            shard = {}
            for k, t in self.tracks.items():
                rows = [i for i, rg in enumerate(per_track[k]) if rg == g]
                if not rows:
                    raise RuntimeError(f"track {k!r} has no samples under root group {g!r}")
                shard[k] = t.select(torch.tensor(rows))
            out.append(type(self)(tracks=shard))
        return out

    def propagate_rewards(self, op: str = "mean") -> "RolloutResp":
        """Fill missing parent rewards from their (single) child track, leaves first."""
        if op not in ("mean", "max", "sum"):
            raise ValueError(f"propagate_rewards: unknown op {op!r}")
        kids: Dict[str, List[str]] = {}
        for k, t in self.tracks.items():
            if t.parent_track is not None:
                kids.setdefault(t.parent_track, []).append(k)

        def depth(k: str) -> int:
            return 1 + max(map(depth, kids[k])) if kids.get(k) else 0

        done: Dict[str, RolloutTrack] = {}
        for k in sorted(self.tracks, key=depth):
            t = self.tracks[k]
            if t.rewards is not None or not kids.get(k):
                done[k] = t
                continue
            if len(kids[k]) > 1:
                raise NotImplementedError(f"track {k!r} has several children {sorted(kids[k])}")
            child = done[kids[k][0]]
            if child.rewards is None:
                raise ValueError(f"child track {kids[k][0]!r} is unscored; score leaves first")
            n_p, n_c = len(t.sample_ids), len(child.sample_ids)
            if n_p == 0 or n_c % n_p:
                raise ValueError(f"non-uniform branching {n_c} → {n_p}")
            grid = hydrate_if_handle(child.rewards).view(n_p, n_c // n_p)
            done[k] = t.replace(rewards={"mean": grid.mean, "max": grid.amax, "sum": grid.sum}[op](dim=1))
        return type(self)(tracks={k: done[k] for k in self.tracks}, reward_compute_s=self.reward_compute_s)


Decoded = Any

__all__ = ["RolloutTrack", "RolloutResp", "Decoded", "hydrate_if_handle"]
