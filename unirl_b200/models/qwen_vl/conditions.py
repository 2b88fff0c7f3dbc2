"""Conditions of the vision-language AR stage: prompt token ids plus PER-SAMPLE lists of image patches and grids.

The image fields are concat-kind lists (one entry per sample, ``None`` for text-only samples) so that select / slice /
concat move them together with the prompt rows; a shared field would keep only the first shard's images when several
rollout workers' conditions are concatenated.  Parity: ``unirl/models/qwen_vl/conditions.py``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field
from unirl_b200.types.conditions import TextTokenCondition


@dataclass
class QwenVLARConditions(Batch):
    prompt: Optional[TextTokenCondition] = concat_field(default=None)
    pixel_values: Optional[List[Any]] = concat_field(default=None)
    image_grid_thw: Optional[List[Any]] = concat_field(default=None)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "QwenVLARConditions":
        p = d.get("prompt")
        if not isinstance(p, TextTokenCondition):
            raise TypeError(f"QwenVLARConditions: d['prompt'] must be a TextTokenCondition, got {type(p).__name__}")
        return cls(prompt=p, pixel_values=d.get("pixel_values"), image_grid_thw=d.get("image_grid_thw"))

    def to_dict(self) -> Dict[str, Any]:
        if self.prompt is None:
            raise ValueError("QwenVLARConditions.to_dict: prompt is None")
        return {"prompt": self.prompt, "pixel_values": self.pixel_values, "image_grid_thw": self.image_grid_thw}

    def extras(self) -> Optional[List[Optional[Dict[str, Any]]]]:
        if self.pixel_values is None:
            return None
        grids = self.image_grid_thw or [None] * len(self.pixel_values)
        return [None if pv is None else {"pixel_values": pv, "image_grid_thw": g} for pv, g in zip(self.pixel_values, grids)]


__all__ = ["QwenVLARConditions"]
