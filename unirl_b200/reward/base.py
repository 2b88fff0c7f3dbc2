"""Reward backend contract + weighted multi-reward combiner.  Parity: ``unirl/reward/base.py:16-79``."""

from __future__ import annotations

import time
from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, Sequence

from unirl_b200.types.reward import RewardRequest, RewardResponse


class RewardBackend(ABC):
    preferred_input_kind: str = "text"  # image | video | text

    @abstractmethod
    def compute_rewards(self, request: RewardRequest) -> RewardResponse: ...

    def get_model_name(self) -> str:
        return type(self).__name__

    def is_available(self) -> bool:
        return True

    def offload(self) -> None:
        pass

    def onload(self) -> None:
        pass

    def dispose(self) -> None:
        pass


class MultiRewardBackend(RewardBackend):
    """``reward = Σ w_i · reward_i``; per-backend values are reported as components."""

    def __init__(self, backends: Dict[str, RewardBackend], weights: Optional[Dict[str, float]] = None):
        if not backends:
            raise ValueError("MultiRewardBackend needs at least one backend")
        self.backends = dict(backends)
        self.weights = {k: float((weights or {}).get(k, 1.0)) for k in self.backends}
        kinds = {b.preferred_input_kind for b in self.backends.values()}
        if len(kinds) > 1:
            raise ValueError(f"MultiRewardBackend mixes input kinds {sorted(kinds)}")
        self.preferred_input_kind = kinds.pop()

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        parts = {k: b.compute_rewards(request) for k, b in self.backends.items()}
        n = len(next(iter(parts.values())).rewards)
        total = [sum(self.weights[k] * parts[k].rewards[i] for k in parts) for i in range(n)]
        ok = [all(parts[k].successes[i] for k in parts) for i in range(n)]
        errs = [next((parts[k].errors[i] for k in parts if parts[k].errors[i]), None) for i in range(n)]
        return RewardResponse(rewards=total, component_rewards={k: list(p.rewards) for k, p in parts.items()}, successes=ok, errors=errs,
                              compute_time=time.perf_counter() - t0)

    def is_available(self) -> bool:
        return all(b.is_available() for b in self.backends.values())


__all__ = ["RewardBackend", "MultiRewardBackend"]
