"""Reward request / response contracts.  Parity: ``unirl/types/reward.py:13-123``."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

from unirl_b200.distributed.tensor.batch import Batch, concat_field, max_field


class RewardType(str, Enum):
    IMAGE_TEXT_ALIGNMENT = "image_text_alignment"
    AESTHETIC = "aesthetic"
    HUMAN_PREFERENCE = "human_preference"
    OCR = "ocr"
    COMPOSITIONAL = "compositional"
    VIDEO_QUALITY = "video_quality"
    TEXT_EXACT_MATCH = "text_exact_match"
    TEXT_MATH = "text_math"
    CUSTOM = "custom"


@dataclass
class RewardRequest:
    primitives: Dict[str, Any] = field(default_factory=dict)
    generated: Dict[str, Any] = field(default_factory=dict)
    metadata: Optional[List[Optional[Dict[str, Any]]]] = None
    prompt_ids: Optional[List[str]] = None
    sample_ids: Optional[List[str]] = None
    group_ids: Optional[List[str]] = None
    reward_types: List[RewardType] = field(default_factory=lambda: [RewardType.IMAGE_TEXT_ALIGNMENT])
    return_components: bool = False

    @property
    def batch_size(self) -> int:
        if self.sample_ids:
            return len(self.sample_ids)
        for v in list(self.generated.values()) + list(self.primitives.values()):
            try:
                return len(v)
            except TypeError:
                continue
        return 0


@dataclass
class RewardResponse(Batch):
    rewards: List[float] = concat_field(default_factory=list)
    component_rewards: Dict[str, List[float]] = concat_field(default_factory=dict)
    successes: List[bool] = concat_field(default_factory=list)
    errors: List[Optional[str]] = concat_field(default_factory=list)
    compute_time: float = max_field(default=0.0)

    @classmethod
    def ok(cls, rewards: List[float], components: Optional[Dict[str, List[float]]] = None, compute_time: float = 0.0) -> "RewardResponse":
        n = len(rewards)
        return cls(rewards=[float(r) for r in rewards], component_rewards=components or {}, successes=[True] * n,
                   errors=[None] * n, compute_time=compute_time)


__all__ = ["RewardType", "RewardRequest", "RewardResponse"]
