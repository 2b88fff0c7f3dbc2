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
        """Fan every prompt out to ``samples_per_prompt`` rows that stay next to each other (the layout group-relative advantages
        expect).  Row ``j`` of the prompt with group id ``<gid>`` is named ``prompt:<gid>:sample:<j>``, the id grammar rewards,
        noise recipes and logs key on; with one sample per prompt the batch is returned unchanged."""
        fan_out = int(samples_per_prompt)
        if fan_out <= 0:
            raise ValueError(f"RolloutInputs.expand: need at least one sample per prompt (got samples_per_prompt={samples_per_prompt!r})")
        if fan_out == 1:
            return self
        widened = self.repeat_interleave(fan_out)
        names: List[str] = []
        for gid in self.group_ids:
            names.extend(f"prompt:{gid}:sample:{j}" for j in range(fan_out))
        widened.sample_ids = names
        return widened


__all__ = ["RolloutInputs"]
