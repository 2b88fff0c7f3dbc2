"""``RolloutInputs`` — what the data source hands the trainer.  Parity: ``unirl/types/prompts.py:11-27``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field


@dataclass
class RolloutInputs(Batch):
    primitives: Dict[str, Any] = concat_field(default_factory=dict)
    sample_ids: List[str] = concat_field(default_factory=list)
    group_ids: List[str] = concat_field(default_factory=list)
    metadata: List[Optional[Dict[str, Any]]] = concat_field(default_factory=list)

    @property
    def batch_size(self) -> int:
        return len(self.sample_ids) if self.sample_ids else super().batch_size

    def expand(self, samples_per_prompt: int) -> "RolloutInputs":
        """Each prompt ``k`` times, siblings adjacent; ids become ``prompt:<gid>:sample:<j>``."""
        k = int(samples_per_prompt)
        if k < 1:
            raise ValueError(f"samples_per_prompt must be >= 1, got {k}")
        if k == 1:
            return self
        out = self.repeat_interleave(k)
        out.sample_ids = [f"prompt:{g}:sample:{j}" for g in self.group_ids for j in range(k)]
        return out


__all__ = ["RolloutInputs"]
