"""Which denoising steps are stochastic (recorded and trained on) for a given rollout.

``AllSDEScheduler`` picks a fraction range of the steps, optionally a random ``num_sde_steps``
subset seeded by the rollout id (``0`` ⇒ forward-process algorithms that need no trajectory);
``WindowScheduler`` slides a window over the schedule (MixGRPO): ``progressive`` advances every
``iters_per_window`` rollouts, ``random`` draws the window start from the rollout id.  Both are
stateless functions of the rollout id, so a resumed job reproduces the same curriculum.
Parity: ``unirl/utils/scheduler_utils.py:86-124``, ``:127-171``, ``:180-218``.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple, Union

import numpy as np


@dataclass
class SchedulerConfig:
    timestep_strategy: str = "all"
    timestep_fraction: Any = 1.0
    num_sde_steps: Optional[int] = None
    window_strategy: str = "progressive"
    window_size: int = 4
    iters_per_window: int = 25
    window_init_timestep: int = 0
    overlap_size: int = 0
    roll_back: bool = False
    max_iters_per_window: Optional[int] = None
    min_iters_per_window: Optional[int] = None


@dataclass
class WindowConfig:
    strategy: str = "all"
    window_size: int = 4
    iters_per_window: int = 25
    init_timestep: int = 0
    overlap_size: int = 0
    roll_back: bool = False
    max_iters_per_window: Optional[int] = None
    min_iters_per_window: Optional[int] = None
    exp_decay_threshold: int = 13
    exp_decay_k: float = 0.1

    def __post_init__(self) -> None:
        if self.strategy == "decay":
            self.max_iters_per_window = self.max_iters_per_window or self.iters_per_window
            self.min_iters_per_window = self.min_iters_per_window or max(1, self.iters_per_window // 4)


class TimestepScheduler(ABC):
    def __init__(self, num_timesteps: int):
        self.num_timesteps = int(num_timesteps)

    @abstractmethod
    def get_sde_indices(self, step: Optional[int] = None) -> Set[int]: ...


def normalize_timestep_fraction(frac: Union[float, Sequence[float]]) -> Tuple[float, float]:
    if isinstance(frac, Sequence) and not isinstance(frac, str):
        if len(frac) != 2:
            raise ValueError(f"timestep_fraction range needs 2 entries, got {len(frac)}")
        lo, hi = float(frac[0]), float(frac[1])
    else:
        lo, hi = 0.0, float(frac)
    if not (0.0 <= lo <= hi <= 1.0):
        raise ValueError(f"timestep_fraction must satisfy 0 <= start <= end <= 1, got ({lo}, {hi})")
    return lo, hi


class AllSDEScheduler(TimestepScheduler):
    def __init__(self, num_timesteps: int, timestep_fraction: Union[float, Sequence[float]] = 1.0, num_sde_steps: Optional[int] = None):
        super().__init__(num_timesteps)
        self.timestep_fraction, self.num_sde_steps = timestep_fraction, num_sde_steps
        lo, hi = normalize_timestep_fraction(timestep_fraction)
        self._lo, self._hi = int(self.num_timesteps * lo), int(self.num_timesteps * hi)
        if num_sde_steps is not None and not 0 <= num_sde_steps <= self._hi - self._lo:
            raise ValueError(f"num_sde_steps={num_sde_steps} outside [0, {self._hi - self._lo}] for steps [{self._lo}, {self._hi})")

    def get_sde_indices(self, step: Optional[int] = None) -> Set[int]:
        if self.num_sde_steps == 0:
            return set()
        pool = list(range(self._lo, self._hi))
        if self.num_sde_steps is None or self.num_sde_steps >= len(pool):
            return set(pool)
        rng = np.random.default_rng(0 if step is None else int(step))
        return {int(i) for i in rng.choice(pool, size=self.num_sde_steps, replace=False)}


class WindowScheduler(TimestepScheduler):
    STRATEGIES = ("all", "progressive", "random")

    def __init__(self, num_timesteps: int, config: WindowConfig):
        super().__init__(num_timesteps)
        if config.strategy not in self.STRATEGIES:
            raise ValueError(f"window strategy {config.strategy!r} not in {self.STRATEGIES}")
        self.config = config

    def get_sde_indices(self, step: Optional[int] = None) -> Set[int]:
        c, step = self.config, 0 if step is None else int(step)
        if c.strategy == "all":
            return set(range(self.num_timesteps))
        if c.strategy == "random":
            start = int(np.random.default_rng(step).integers(0, max(0, self.num_timesteps - c.window_size) + 1))
            return set(range(start, start + c.window_size))
        stride = c.window_size - c.overlap_size
        rounds = max(1, (self.num_timesteps - c.init_timestep - c.window_size) // stride + 1)
        w = step // c.iters_per_window
        w = w % rounds if c.roll_back else min(w, rounds - 1)
        start = c.init_timestep + w * stride
        return set(range(start, start + c.window_size))


SCHEDULER_REGISTRY = {"all": AllSDEScheduler, "window": WindowScheduler}


def create_indices_scheduler(*, scheduler_config: Union[SchedulerConfig, Dict[str, Any]], num_timesteps: int) -> TimestepScheduler:
    get = scheduler_config.get if isinstance(scheduler_config, dict) else (lambda k, d=None: getattr(scheduler_config, k, d))
    kind = str(get("timestep_strategy", "all"))
    if kind == "all":
        return AllSDEScheduler(int(num_timesteps), get("timestep_fraction", 1.0), get("num_sde_steps", None))
    if kind == "window":
        return WindowScheduler(int(num_timesteps), WindowConfig(
            strategy=get("window_strategy", "progressive"), window_size=int(get("window_size", 4)),
            iters_per_window=int(get("iters_per_window", 25)), init_timestep=int(get("window_init_timestep", 0)),
            overlap_size=int(get("overlap_size", 0)), roll_back=bool(get("roll_back", False)),
            max_iters_per_window=get("max_iters_per_window", None), min_iters_per_window=get("min_iters_per_window", None)))
    raise ValueError(f"unknown timestep_strategy {kind!r} (have {sorted(SCHEDULER_REGISTRY)})")


__all__ = ["SchedulerConfig", "WindowConfig", "TimestepScheduler", "AllSDEScheduler", "WindowScheduler",
           "normalize_timestep_fraction", "create_indices_scheduler", "SCHEDULER_REGISTRY"]
