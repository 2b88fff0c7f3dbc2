"""Exponential moving averages of the trainable weights.

Full-weight EMA keeps an fp32 shadow per optimizer shard, updated inside the fused AdamW kernel
(``timing="optimizer_step"``) or by one lerp per group at rollout end.  ``apply_shadow`` /
``restore_shadow`` swap the shadow into the bf16 replica for EMA rollouts / evaluation and
``use_shadow()`` is the context manager DiffusionNFT uses for its "old" policy.
Decay schedules: ``constant``, ``linear`` (ramp over ``flat_steps``), ``warmup`` and the default
``min((1+t)/(10+t), target)``.  Parity: ``unirl/train/ema.py:17-83``.
"""

from __future__ import annotations

import contextlib
from typing import Any, Iterator, List, Optional

import torch


def ema_decay_at(t: int, target: float, kind: str = "default", flat_steps: int = 0, uprate: float = 0.001, uphold: float = 0.5) -> float:
    if kind == "constant":
        return target
    if kind == "linear":
        return target if flat_steps <= 0 else min(target, target * (t + 1) / flat_steps)
    if kind == "warmup":
        return min(uphold, uprate * max(0, t - flat_steps)) if t >= flat_steps else 0.0
    return min((1.0 + t) / (10.0 + t), target)


class ShardEMA:
    """EMA over the fp32 master shards of a :class:`FlatShardedModel`."""

    def __init__(self, sharded: Any, target_decay: float = 0.9999, timing: str = "optimizer_step", decay_type: str = "default", **decay_kw: Any):
        self.sharded, self.target_decay, self.timing, self.decay_type, self.decay_kw = sharded, float(target_decay), timing, decay_type, decay_kw
        for g in sharded.groups:
            g.ema = g.master.float().clone() if g.trainable else None
        self._stash: Optional[List[torch.Tensor]] = None

    def decay(self, t: int) -> float:
        return ema_decay_at(t, self.target_decay, self.decay_type, **self.decay_kw)

    def _lerp(self, t: int) -> None:
        d = self.decay(t)
        for g in self.sharded.groups:
            if g.ema is not None:
                g.ema.mul_(d).add_(g.master.float(), alpha=1.0 - d)

    def step(self, t: int) -> None:
        if self.timing == "optimizer_step":
            self._lerp(t)

    def on_rollout_end(self, t: int) -> None:
        if self.timing == "rollout_end":
            self._lerp(t)

    def apply_shadow(self) -> None:
        if self._stash is not None:
            return
        self._stash = []
        for g in self.sharded.groups:
            if g.ema is None:
                continue
            self._stash.append(g.param_shard.clone())
            g.param_shard.copy_(g.ema.to(g.param_shard.dtype))
            self.sharded.shard_comm.publish_params(g)

    def restore_shadow(self) -> None:
        if self._stash is None:
            return
        it = iter(self._stash)
        for g in self.sharded.groups:
            if g.ema is None:
                continue
            g.param_shard.copy_(next(it))
            self.sharded.shard_comm.publish_params(g)
        self._stash = None

    @contextlib.contextmanager
    def use_shadow(self) -> Iterator[None]:
        self.apply_shadow()
        try:
            yield
        finally:
            self.restore_shadow()


__all__ = ["ShardEMA", "ema_decay_at"]
