"""Selective trajectory storage: keep only the latents an algorithm will replay.

For SDE step ``i`` the replay needs the pair ``(x_i, x_{i+1})``; everything else is dropped while
sampling, which is what keeps 32 k-token video rollouts resident in HBM.  Parity:
``unirl/types/trajectory_store.py:16-248``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, List, Set, Tuple

import torch

from unirl_b200.distributed.tensor.batch import Batch, concat_field, shared_field


def compute_trajectory_positions(sde_indices: Iterable[int], num_steps: int) -> List[int]:
    """Sorted positions covering ``(i, i+1)`` for each SDE step, clamped to ``[0, num_steps]``."""
    clamp = lambda p: max(0, min(int(p), num_steps))  # noqa: E731
    return sorted({clamp(i + d) for i in sde_indices for d in (0, 1)})


def _index_map(positions: List[int], total: int) -> torch.Tensor:
    m = torch.full((total,), -1, dtype=torch.long)
    for slot, pos in enumerate(positions):
        if 0 <= pos < total:
            m[pos] = slot
    return m


@dataclass
class Trajectory(Batch):
    """``data[B, K, …]`` holds K stored positions; ``index_map[pos]`` is the slot or -1."""

    data: torch.Tensor = concat_field(default=None)
    index_map: torch.Tensor = shared_field(default=None)
    total_positions: int = shared_field(default=0)

    @classmethod
    def from_full(cls, traj: torch.Tensor) -> "Trajectory":
        n = int(traj.shape[1])
        return cls(traj, torch.arange(n), n)

    @classmethod
    def from_clean_latents(cls, clean: torch.Tensor, total_positions: int = 1) -> "Trajectory":
        return cls(clean.unsqueeze(1), _index_map([total_positions - 1], total_positions), total_positions)

    @classmethod
    def from_selective(cls, traj: torch.Tensor, collected_positions: List[int], total_positions: int) -> "Trajectory":
        if int(traj.shape[1]) != len(collected_positions):
            raise ValueError(f"{traj.shape[1]} stored slots vs {len(collected_positions)} positions")
        return cls(traj, _index_map(list(collected_positions), total_positions), total_positions)

    @property
    def batch_size(self) -> int:
        return int(self.data.shape[0])

    @property
    def num_stored(self) -> int:
        return int(self.data.shape[1])

    @property
    def device(self) -> torch.device:
        return self.data.device

    @property
    def is_full(self) -> bool:
        return self.num_stored == self.total_positions

    @property
    def is_clean_latents_only(self) -> bool:
        return self.num_stored == 1

    @property
    def is_selective(self) -> bool:
        return not self.is_full and not self.is_clean_latents_only

    @property
    def stored_positions(self) -> List[int]:
        return (self.index_map >= 0).nonzero().flatten().tolist()

    @property
    def clean_latents(self) -> torch.Tensor:
        return self.data[:, int(self.index_map[self.stored_positions[-1]])]

    def has_position(self, pos: int) -> bool:
        return 0 <= pos < self.total_positions and int(self.index_map[pos]) >= 0

    def get_position(self, pos: int) -> torch.Tensor:
        if not 0 <= pos < self.total_positions:
            raise IndexError(f"position {pos} outside [0, {self.total_positions})")
        slot = int(self.index_map[pos])
        if slot < 0:
            raise IndexError(f"position {pos} was not stored (stored: {self.stored_positions})")
        return self.data[:, slot]

    def get_pair(self, pos: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.get_position(pos), self.get_position(pos + 1)

    def slice_batch(self, start: int, end: int) -> "Trajectory":
        return Trajectory(self.data[start:end].clone(), self.index_map, self.total_positions)

    def index_select_batch(self, idx: torch.Tensor) -> "Trajectory":
        return self.select(idx)

    reindex_batch = index_select_batch

    def cast_dtype(self, dtype: torch.dtype) -> "Trajectory":
        if self.data.is_floating_point() and self.data.dtype != dtype:
            return Trajectory(self.data.to(dtype), self.index_map, self.total_positions)
        return self

    def detect_modality(self) -> str:
        return "video" if self.data.ndim >= (6 if self.is_full else 5) else "image"


class TrajectoryBuilder:
    """Collects latents during a denoising loop, silently dropping positions nobody asked for."""

    def __init__(self, total_steps: int, needed_positions: Set[int]):
        self.total_steps = total_steps
        self.needed = set(needed_positions)
        self._slots: List[Tuple[int, torch.Tensor]] = []

    @classmethod
    def for_sde_steps(cls, sde_indices: Iterable[int], total_steps: int) -> "TrajectoryBuilder":
        return cls(total_steps, set(compute_trajectory_positions(sde_indices, total_steps)) or {total_steps})

    @classmethod
    def full(cls, total_steps: int) -> "TrajectoryBuilder":
        return cls(total_steps, set(range(total_steps + 1)))

    def add(self, position: int, latents: torch.Tensor) -> None:
        if position in self.needed:
            self._slots.append((position, latents))

    def finalize(self) -> Trajectory:
        if not self._slots:
            raise ValueError(f"no positions collected (needed {sorted(self.needed)})")
        total = self.total_steps + 1
        return Trajectory(torch.stack([t for _, t in self._slots], 1), _index_map([p for p, _ in self._slots], total), total)


TrajectoryStore = Trajectory

__all__ = ["Trajectory", "TrajectoryBuilder", "TrajectoryStore", "compute_trajectory_positions"]
