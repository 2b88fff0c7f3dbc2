"""Per-phase timings of a rollout step and the derived throughput figures.  Parity: ``unirl/utils/timing.py:19-55``."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional


@dataclass
class PhaseTimings:
    phases: Dict[str, float] = field(default_factory=dict)
    step_time_s: float = 0.0

    def add(self, name: str, seconds: float) -> None:
        self.phases[name] = self.phases.get(name, 0.0) + float(seconds)

    def as_perf_dict(self, num_samples: Optional[int] = None, num_tokens: Optional[int] = None) -> Dict[str, float]:
        out = {f"perf/{k}_time_s": v for k, v in self.phases.items()}
        out["perf/step_time_s"] = self.step_time_s
        if self.step_time_s > 0:
            if num_samples:
                out["perf/samples_per_s"] = num_samples / self.step_time_s
            if num_tokens:
                out["perf/tokens_per_s"] = num_tokens / self.step_time_s
        return out


__all__ = ["PhaseTimings"]
