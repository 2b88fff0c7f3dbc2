"""Typed conditions of the Qwen3 AR stage: one ``prompt`` slot of token ids.  Parity: ``unirl/models/qwen3/conditions.py``."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.types.conditions import Condition, TextTokenCondition


@dataclass
class Qwen3ARConditions(Batch):
    prompt: Optional[TextTokenCondition] = concat_field(default=None)

    @classmethod
    def from_dict(cls, d: Dict[str, Condition]) -> "Qwen3ARConditions":
        p = d.get("prompt")
        if not isinstance(p, TextTokenCondition):
            raise TypeError(f"Qwen3ARConditions: d['prompt'] must be a TextTokenCondition, got {type(p).__name__}")
        return cls(prompt=p)

    def to_dict(self) -> Dict[str, Condition]:
        if self.prompt is None:
            raise ValueError("Qwen3ARConditions.to_dict: prompt is None")
        return {"prompt": self.prompt}


__all__ = ["Qwen3ARConditions"]
