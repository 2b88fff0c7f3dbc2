"""LR schedules (constant / linear / cosine with warm-up) as pure functions of the optimizer step.

The optimizer itself is the fused flat-shard AdamW of ``parallel/flat_shard.py``; this module only
supplies the multiplier.  Parity: ``unirl/train/factories.py:21-104``.
"""

from __future__ import annotations

import math
from typing import Any, Dict

from unirl_b200.train.configs import LrSchedulerConfig


class LrSchedule:
    def __init__(self, cfg: LrSchedulerConfig, base_lr: float):
        self.cfg, self.base_lr = cfg, float(base_lr)
        self.step_count = 0
        if cfg.type not in ("constant", "linear", "cosine"):
            raise ValueError(f"unknown lr schedule '{cfg.type}'")

    def multiplier(self, step: int) -> float:
        c = self.cfg
        if c.warmup_steps > 0 and step < c.warmup_steps:
            return (step + 1) / c.warmup_steps
        if c.type == "constant":
            return 1.0
        span = max(1, c.total_steps - c.warmup_steps)
        frac = min(1.0, max(0.0, (step - c.warmup_steps) / span))
        return 1.0 - frac if c.type == "linear" else 0.5 * (1.0 + math.cos(math.pi * frac))

    @property
    def lr(self) -> float:
        return self.base_lr * self.multiplier(self.step_count)

    def step(self) -> None:
        self.step_count += 1

    def state_dict(self) -> Dict[str, Any]:
        return {"last_epoch": self.step_count, "base_lrs": [self.base_lr], "_step_count": self.step_count + 1}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = int(sd.get("last_epoch", 0))


def build_lr_scheduler(cfg: LrSchedulerConfig, base_lr: float) -> LrSchedule:
    return LrSchedule(cfg, base_lr)


__all__ = ["LrSchedule", "build_lr_scheduler"]
